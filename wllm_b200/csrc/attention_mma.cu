// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16,
// 32-bit accumulation), compiled for one head size: -DHEAD_DIM=<multiple of 16, <= 256>.
//
// Two kernels share the tile code.
//
//   decode   one CTA per (request with one new token, kv head, split of its keys).  The
//            query heads of the kv head's group are the rows of one 16-row tile, so the
//            keys are read once for the whole group.  Head sizes in steps of 64 run the
//            warp-specialised kernel (a TMA producer warp, three consumer warps that take
//            whole 32-key tiles in turn); other head sizes run four warps that take 16-key
//            slices of every 64-key tile.  The warps merge at the end.  Splits of
//            `split_keys` keys give a long context to many SMs; each writes its partial
//            (max, sum, unnormalised output) to scratch and a second kernel merges them
//            in split order.  A request with a single split writes its output directly.
//            (Letting the CTA that finishes last merge them inside the kernel was built and
//            measured: a gain of 1% at first, a loss of 4% once the kernels around it had
//            become shorter; the merge kernel spreads over 64 CTAs what one CTA did alone.)
//   prefill  one CTA per (request with several new tokens, kv head, tile of 128 rows),
//            rows = (token, query head of the group).  Head sizes in steps of 64 run on
//            tcgen05 (scores and output accumulate in tensor memory: attention_prefill_tc.cuh);
//            other head sizes on mma.sync: eight warps own 16 rows each and walk all 64-key
//            tiles up to the causal edge.
//
// Keys and values come straight from the pages through the request's block table
// ([page][kv_head][slot][head_dim] layout) into a swizzled multi-stage ring in shared memory.
// Head sizes that are multiples of 64: one thread issues TMA box copies (cp.async.bulk.tensor,
// 128-byte swizzle, 64 columns x up to 64 slots of one page and head per box) that complete on an
// mbarrier; rows past a request's keys hold whatever the page holds and are masked.  Other head
// sizes: 16-byte cp.async by all threads, rows outside a request's keys zero-filled.
// Waits on the mbarriers are bounded; a CTA that gives up records a code in `status` and leaves.
// Scores, the running maximum and sum and the output accumulate in 32-bit; the
// exponentials are exp2 of log2(e)-scaled scores.  Which requests each kernel serves is
// read from q_len on the device (1: decode, more: prefill), so a captured graph stays
// valid when the batch changes its contents but not its shape.
#include "tc_common.cuh"

#include <mutex>
#include <unordered_map>

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
constexpr bool USE_TMA = (HD % 64 == 0);
constexpr int SPLIT_TILE = USE_TMA ? 32 : BN;    // the decode kernels' key tile: splits are whole tiles of it
enum { GAVE_UP_DECODE = 21, GAVE_UP_PREFILL = 22 };

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile of ROWS rows.  cp.async layout: rows of
// ROWB bytes, chunks XOR-swizzled inside each 128-byte group.  TMA layout: one sub-tile [ROWS][128 bytes]
// per 64 columns (what a 128-byte-swizzled box copy writes), the same XOR inside each 128-byte row.
template <int ROWS>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    if (USE_TMA) return (uint32_t)((chunk >> 3) * (ROWS * 128) + row * 128 + ((((chunk ^ row) & 7)) << 4));
    return (uint32_t)(row * ROWB + ((((chunk & ~7) | ((chunk ^ row) & 7))) << 4));
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return smem_addr(p); }
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

// Rows [row_lo, row_hi) of a value tile of ROWS rows in the box-copy layout (`blocks` column blocks of
// [ROWS][128 bytes]) set to zero, by `nthreads` threads of which this is number `tid`.  A box copy brings whole
// rows of a page: behind a request's last key, and in front of a window's first, they hold whatever the page
// holds.  Such keys get a weight of zero, but the product 0 x v is no zero when v is not a number, so their
// values are cleared in the few tiles that reach past either end.
template <int ROWS>
__device__ __forceinline__ void zero_value_rows(uint32_t v_tile, int blocks, int row_lo, int row_hi, int tid, int nthreads) {
    const int per_row = blocks * 8;
    for (int i = tid; i < (row_hi - row_lo) * per_row; i += nthreads) {
        const int row = row_lo + i / per_row, rest = i % per_row;
        const uint32_t addr = v_tile + (rest >> 3) * (ROWS * 128) + row * 128 + (rest & 7) * 16;
        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
    }
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
        cp_async16(k_dst + swz<BN>(row, chunk), k_pages + off, valid);
        cp_async16(v_dst + swz<BN>(row, chunk), v_pages + off, valid);
    }
}

// The same tile by TMA (one thread): per page that the tile touches and per 64 columns, one box of
// [min(page_size, 64) slots][64 columns] of keys and one of values.  The pool is seen as a matrix of
// [pages * nkv * page_size rows][HD columns]; a released or unallocated page (< 0) is read as page 0 and masked.
__device__ __forceinline__ void tma_kv_tile(uint32_t k_dst, uint32_t v_dst, uint32_t bar, const CUtensorMap* k_map,
                                            const CUtensorMap* v_map, const int* __restrict__ table, int max_pages,
                                            int tile_start, int g, int nkv, int page_size, int page_shift) {
    mbar_expect_tx(bar, 2 * TILE_BYTES);
    const int box_rows = page_size < BN ? page_size : BN;
    for (int r0 = 0; r0 < BN; r0 += box_rows) {
        const int key = tile_start + r0;
        const int index = key >> page_shift;          // the last tile may reach past the request's pages
        int page = index < max_pages ? table[index] : 0;
        if (page < 0) page = 0;
        const int row = (page * nkv + g) * page_size + (key & (page_size - 1));
#pragma unroll
        for (int cb = 0; cb < HD / 64; ++cb) {
            tma_load_2d(k_dst + cb * (BN * 128) + r0 * 128, k_map, bar, cb * 64, row);
            tma_load_2d(v_dst + cb * (BN * 128) + r0 * 128, v_map, bar, cb * 64, row);
        }
    }
}

// Rows of the query tile: row m of a (request, kv head) is (token m / rep, head g*rep + m % rep).
template <int NT, int ROWS>
__device__ __forceinline__ void load_q_tile(uint32_t dst, const bf16* __restrict__ q, int q_stride, int q_start, int q_len,
                                            int row0, int nrows, int g, int rep) {
    for (int idx = threadIdx.x; idx < nrows * CPR; idx += NT) {
        const int row = idx / CPR, chunk = idx % CPR;
        const int m = row0 + row;
        const bool valid = m < q_len * rep;
        const bf16* src = q;
        if (valid) src = q + (size_t)(q_start + m / rep) * q_stride + (size_t)(g * rep + m % rep) * HD + chunk * 8;
        cp_async16(dst + swz<ROWS>(row, chunk), src, valid);
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
template <int NKEYS, int QROWS, int KROWS = BN>
__device__ __forceinline__ void warp_tile(RowState& st, uint32_t q_tile, int q_row0, uint32_t k_tile, uint32_t v_tile, int key0,
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
        ldsm4(q_tile + swz<QROWS>(q_row0 + a_row, kt * 2 + a_chunk), a);
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            uint32_t b[4];
            ldsm4(k_tile + swz<KROWS>(key0 + np * 16 + b_row, kt * 2 + b_chunk), b);
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
            ldsm4t(v_tile + swz<KROWS>(key0 + kk * 16 + v_row, np * 2 + v_chunk), b);
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
// the tile ring: cp.async groups, or TMA with one "full" mbarrier per stage
// --------------------------------------------------------------------------------------
// Both kernels walk tiles t0 .. t1-1 with the same schedule: before tile t is used, every thread waits
// until it has landed, then the CTA synchronises (so tile t-1's stage is free) and the load of tile
// t + STAGES - 1 is issued into that stage.
template <int STAGES, int NT>
struct TileRing {
    uint32_t kv_s, bars;          // shared-memory addresses of the stages and of the mbarriers
    const bf16 *k_pages, *v_pages;
    const CUtensorMap *k_map, *v_map;
    const int* table;
    int max_pages, key_lo, key_hi, g, nkv, page_size, page_shift, t0, t1;
    int ctx_end;                  // the request's keys end here: rows of a box copy from here on hold no key

    __device__ __forceinline__ uint32_t k_stage(int s) const { return kv_s + (2 * s) * TILE_BYTES; }
    __device__ __forceinline__ uint32_t v_stage(int s) const { return kv_s + (2 * s + 1) * TILE_BYTES; }

    __device__ __forceinline__ void init() {
        if (USE_TMA) {
            if (threadIdx.x == 0) {
                for (int s = 0; s < STAGES; ++s) mbar_init(bars + 8 * s, 1);
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            __syncthreads();
        }
    }
    __device__ __forceinline__ void issue(int t) {      // tile t into its stage
        const int s = (t - t0) % STAGES;
        if (USE_TMA) {
            if (threadIdx.x == 0 && t < t1)
                tma_kv_tile(k_stage(s), v_stage(s), bars + 8 * s, k_map, v_map, table, max_pages, t * BN, g, nkv, page_size,
                            page_shift);
        } else {
            if (t < t1)
                load_kv_tile<NT>(k_stage(s), v_stage(s), k_pages, v_pages, table, t * BN, key_lo, key_hi, g, nkv, page_size,
                                 page_shift);
            cp_commit();
        }
    }
    __device__ __forceinline__ void prologue() {
        for (int s = 0; s < STAGES - 1; ++s) issue(t0 + s);
    }
    // false (for every thread of the CTA alike) if the tile did not arrive within the limit (TMA only)
    __device__ __forceinline__ bool arrive(int t) {
        int ok = 1;
        if (USE_TMA) {
            const int n = t - t0;
            ok = mbar_wait(bars + 8 * (n % STAGES), (n / STAGES) & 1) ? 1 : 0;
            if (ok && t * BN + BN > ctx_end)
                zero_value_rows<BN>(v_stage(n % STAGES), HD / 64, max(0, ctx_end - t * BN), BN, threadIdx.x, NT);
            if (ok && t * BN < key_lo)
                zero_value_rows<BN>(v_stage(n % STAGES), HD / 64, 0, min(BN, key_lo - t * BN), threadIdx.x, NT);
        } else {
            cp_wait<STAGES - 2>();
        }
        ok = __syncthreads_and(ok);
        if (ok) issue(t + STAGES - 1);
        return ok != 0;
    }
    // Nothing of this CTA's copies may be in flight when it leaves.  After a normal run that is so already;
    // after giving up on tile `failed`, the tiles issued behind it are waited for, again with the limit.
    __device__ __forceinline__ void drain(int failed) {
        if (USE_TMA) {
            for (int t = failed + 1; failed >= 0 && t < min(t1, failed + STAGES - 1); ++t) {
                const int n = t - t0;
                if (!mbar_wait(bars + 8 * (n % STAGES), (n / STAGES) & 1)) break;
            }
        } else {
            cp_wait<0>();
        }
        __syncthreads();
    }
};

// --------------------------------------------------------------------------------------
// decode: grid (max_splits, nkv, requests)
// --------------------------------------------------------------------------------------
constexpr int DEC_STAGES = 3;
constexpr int DEC_SMEM = 1024 + 16 * ROWB + DEC_STAGES * 2 * TILE_BYTES + 64;

// Keys per split of one request.  The launch fixes the number of splits and a planned size (from the longest
// context it may see: under a captured graph that is the reach of the block table).  When the whole grid is
// resident at once (at most one CTA an SM), each request cuts its own keys evenly over its splits, in whole
// tiles, so that a request shorter than the bound does not fill its first split and starve the rest; but not
// in parts below 512 keys (or the planned size, if that is smaller): a CTA's fixed cost is worth about that
// many.  A grid of more CTAs than SMs keeps the planned size: the host chose it so that the short rests,
// which start last, fill the second round; a context longer than planned size x splits (a caller's mistake:
// it cannot see the lengths on the device) widens the parts instead of dropping keys.
// (`split_keys` arrives negated when the grid is resident at once: the host knows, and the merge kernel, whose
// grid differs, has to cut the same way.)
__device__ __forceinline__ int keys_per_split(int ctx, int split_keys, int max_splits, int tile) {
    const int even = ((ctx + max_splits - 1) / max_splits + tile - 1) / tile * tile;
    if (split_keys > 0) return max(split_keys, even);   // never more splits than the launch has CTAs and slots for
    split_keys = -split_keys;
    return max(min(split_keys, 512), even);
}

__global__ void __launch_bounds__(NTHREADS)
decode_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
              const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
              const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
              const int* __restrict__ req_q_start, const int* __restrict__ req_q_len, const int* __restrict__ req_ctx_len,
              const int* __restrict__ block_table, int max_pages, int nq, int nkv, int page_size, int window, float scale2,
              int split_keys, int max_splits, float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    pdl_begin();
    const int split = blockIdx.z, g = blockIdx.y, r = blockIdx.x;     // CTAs start request by request, the last (shortest) splits last
    if (req_q_len[r] != 1) return;
    const int ctx = req_ctx_len[r], pos = ctx - 1;
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int part_keys = keys_per_split(ctx, split_keys, max_splits, SPLIT_TILE);
    const int num_splits = (ctx + part_keys - 1) / part_keys;
    if (split >= num_splits) return;
    const int key_lo = max(split * part_keys, first), key_hi = min(ctx, (split + 1) * part_keys);
    const int rep = nq / nkv, token = req_q_start[r];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // stages at a 1024-byte boundary (swizzle atoms of the box copies), then the query tile, then barriers
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t q_s = base + DEC_STAGES * 2 * TILE_BYTES;

    RowState st;
    init_state(st);
    const bool empty = key_lo >= key_hi;     // the window starts behind this split
    TileRing<DEC_STAGES, NTHREADS> ring;
    ring.kv_s = base; ring.bars = q_s + 16 * ROWB;
    ring.k_pages = k_pages; ring.v_pages = v_pages; ring.k_map = &k_map; ring.v_map = &v_map;
    ring.table = block_table + (size_t)r * max_pages; ring.max_pages = max_pages;
    ring.key_lo = key_lo; ring.key_hi = key_hi; ring.g = g; ring.nkv = nkv; ring.page_size = page_size;
    ring.page_shift = 31 - __clz(page_size);
    ring.t0 = key_lo / BN; ring.t1 = empty ? ring.t0 : (key_hi + BN - 1) / BN;
    ring.ctx_end = ctx;
    ring.init();
    load_q_tile<NTHREADS, 16>(q_s, q, q_stride, token, 1, 0, 16, g, rep);
    if (USE_TMA) cp_commit();
    ring.prologue();
    if (USE_TMA) cp_wait<0>();               // the query tile (cp.async); the first arrive() synchronises the CTA
    const int first_r[2] = {key_lo, key_lo};
    const int hi_r[2] = {min(pos, key_hi - 1), min(pos, key_hi - 1)};
    int t = ring.t0;
    bool ok = true;
    for (; t < ring.t1; ++t) {
        if (!ring.arrive(t)) { ok = false; break; }
        const int s = (t - ring.t0) % DEC_STAGES;
        warp_tile<16, 16>(st, q_s, 0, ring.k_stage(s), ring.v_stage(s), warp * 16, t * BN, hi_r, first_r, scale2);
    }
    ring.drain(ok ? -1 : t);
    if (!ok) {
        if (threadIdx.x == 0) atomicExch(status, GAVE_UP_DECODE);
        return;
    }

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
        const float mbase = M == -INFINITY ? 0.f : M;
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            const float f = exp2f(sm_ml[(w * 16 + row) * 2] - mbase);
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

// --------------------------------------------------------------------------------------
// decode, warp-specialised (head sizes in steps of 64): grid (max_splits, nkv, requests)
// --------------------------------------------------------------------------------------
// One producer warp and six consumer warps.  The producer's elected lane walks the split's keys in
// tiles of 32 and fills a ring of six stages with TMA box copies (keys and values of one tile per stage);
// tile n goes to consumer warp n % 6, which waits for it on the stage's "full" mbarrier, runs all 16
// query rows against its 32 keys, and hands the stage back through the "empty" mbarrier.  No barrier
// spans the CTA until the running states are merged at the end, so a warp that waits for memory or for
// a dependent instruction stalls nobody else, and several tiles are in flight behind those in use.
// The number of stages is a multiple of the number of consumers, so a stage is always served by the
// same warp: a parity wait tells only the current phase from the one before it, and a warp that saw
// every second fill of a stage could take an old phase for the one it is waiting for.
constexpr int WS_BN = 32;
static_assert(!USE_TMA || SPLIT_TILE == WS_BN, "splits are whole tiles of the kernel that runs");
constexpr int MERGE_MAX_SPLITS = 256;
constexpr int WS_STAGES = 6;
constexpr int WS_PAGE_IDS = 256;        // page numbers of a split kept in shared memory (16,384 keys of 64 a page)
constexpr int WS_CONSUMERS = 6;
static_assert(WS_STAGES % WS_CONSUMERS == 0, "every stage must belong to one consumer warp");
constexpr int WS_TILE_BYTES = WS_BN * ROWB;
constexpr int WS_THREADS = (1 + WS_CONSUMERS) * 32;
constexpr int WS_SMEM = 1024 + WS_STAGES * 2 * WS_TILE_BYTES + 16 * ROWB + 128;

__global__ void __launch_bounds__(WS_THREADS)
decode_ws_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                 const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                 const int* __restrict__ req_q_start, const int* __restrict__ req_q_len, const int* __restrict__ req_ctx_len,
                 const int* __restrict__ block_table, int max_pages, int nq, int nkv, int page_size, int window, float scale2,
                 int split_keys, int max_splits, float* __restrict__ part_o, float* __restrict__ part_ml,
                 int whole_rows, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    pdl_launch_dependents();
    // The step's index arrays were copied before its first kernel started, and no kernel of this step writes
    // a key below the new token's place: they may be read before this kernel waits for its predecessor.
    const int split = blockIdx.z, g = blockIdx.y, r = blockIdx.x;     // CTAs start request by request, the last (shortest) splits last
    if (req_q_len[r] != 1) return;
    const int ctx = req_ctx_len[r], pos = ctx - 1;
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int part_keys = keys_per_split(ctx, split_keys, max_splits, SPLIT_TILE);
    const int num_splits = (ctx + part_keys - 1) / part_keys;
    if (split >= num_splits) return;
    const int key_lo = max(split * part_keys, first), key_hi = min(ctx, (split + 1) * part_keys);
    const int rep = nq / nkv, token = req_q_start[r];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t q_s = base + WS_STAGES * 2 * WS_TILE_BYTES;
    const uint32_t full0 = q_s + 16 * ROWB, empty0 = full0 + 8 * WS_STAGES;
    const int* table = block_table + (size_t)r * max_pages;
    const int page_shift = 31 - __clz(page_size);
    const int t0 = key_lo / WS_BN, t1 = key_lo >= key_hi ? t0 : (key_hi + WS_BN - 1) / WS_BN;
    const int box_rows = page_size < WS_BN ? page_size : WS_BN;

    __shared__ int page_ids[WS_PAGE_IDS];
    const int page_lo = (t0 * WS_BN) >> page_shift, page_hi = t1 > t0 ? ((t1 * WS_BN - 1) >> page_shift) + 1 : page_lo;

    // one tile of keys and values into stage s (the producer lane calls this); a step reads them once
    const uint64_t stream = l2_evict_first();
    auto load_tile = [&](int t, int s) {
        const uint32_t k_dst = base + (2 * s) * WS_TILE_BYTES, v_dst = k_dst + WS_TILE_BYTES, bar = full0 + 8 * s;
        mbar_expect_tx(bar, 2 * WS_TILE_BYTES);
        for (int r0 = 0; r0 < WS_BN; r0 += box_rows) {
            const int key = t * WS_BN + r0, index = key >> page_shift;
            int page = index - page_lo < WS_PAGE_IDS ? page_ids[index - page_lo] : (index < max_pages ? table[index] : 0);
            if (page < 0) page = 0;
            const int row = (page * nkv + g) * page_size + (key & (page_size - 1));
            if (whole_rows) {          // one box a tile: the maps have the column blocks as a third dimension
                tma_load_3d_hint(k_dst, &k_map, bar, 0, row, 0, stream);
                tma_load_3d_hint(v_dst, &v_map, bar, 0, row, 0, stream);
                continue;
            }
#pragma unroll
            for (int cb = 0; cb < HD / 64; ++cb) {
                tma_load_2d_hint(k_dst + cb * (WS_BN * 128) + r0 * 128, &k_map, bar, cb * 64, row, stream);
                tma_load_2d_hint(v_dst + cb * (WS_BN * 128) + r0 * 128, &v_map, bar, cb * 64, row, stream);
            }
        }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < WS_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // The page numbers of this split come in with one round of loads by all threads, so that no tile's copy
    // waits for a load of its own in the producer lane.
    for (int i = threadIdx.x; i < min(WS_PAGE_IDS, page_hi - page_lo); i += WS_THREADS)
        page_ids[i] = page_lo + i < max_pages ? table[page_lo + i] : 0;
    __syncthreads();
    // Tiles that end below the new token's place hold only keys of earlier steps: the first stages are
    // requested now, while the kernel that writes the new key and value (and the query) still runs.
    int early = 0;
    if (warp == WS_CONSUMERS && lane == 0) {
        early = max(0, min(WS_STAGES, min(t1, pos / WS_BN) - t0));
        for (int n = 0; n < early; ++n) load_tile(t0 + n, n);
    }
    pdl_wait();
    load_q_tile<WS_THREADS, 16>(q_s, q, q_stride, token, 1, 0, 16, g, rep);
    cp_commit();
    cp_wait<0>();
    __syncthreads();

    RowState st;
    init_state(st);
    bool ok = true;
    if (warp == WS_CONSUMERS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int n = early;
            for (int t = t0 + early; t < t1; ++t, ++n) {
                const int s = n % WS_STAGES;
                if (!mbar_wait(empty0 + 8 * s, ((n / WS_STAGES) & 1) ^ 1)) { ok = false; break; }
                load_tile(t, s);
            }
            // stay until the consumers have handed back every stage that was filled (a stage that was
            // never filled passes at once), so that nothing is in flight when the CTA leaves
            for (int k = 0; k < WS_STAGES && ok; ++k, ++n) {
                const int s = n % WS_STAGES;
                if (!mbar_wait(empty0 + 8 * s, ((n / WS_STAGES) & 1) ^ 1)) ok = false;
            }
            if (!ok) atomicExch(status, GAVE_UP_DECODE);
        }
    } else {
        // ---------------- consumers: warp w takes tiles w, w + 6, ... ----------------
        const int first_r[2] = {key_lo, key_lo};
        const int hi_r[2] = {min(pos, key_hi - 1), min(pos, key_hi - 1)};
        for (int n = warp; t0 + n < t1; n += WS_CONSUMERS) {
            const int s = n % WS_STAGES;
            if (!mbar_wait(full0 + 8 * s, (n / WS_STAGES) & 1)) { ok = false; break; }
            __syncwarp();
            const uint32_t k_src = base + (2 * s) * WS_TILE_BYTES;
            const int tile_start = (t0 + n) * WS_BN;
            if (tile_start + WS_BN > ctx || tile_start < key_lo) {      // rows that hold no key of this request
                if (tile_start + WS_BN > ctx)
                    zero_value_rows<WS_BN>(k_src + WS_TILE_BYTES, HD / 64, max(0, ctx - tile_start), WS_BN, lane, 32);
                if (tile_start < key_lo)
                    zero_value_rows<WS_BN>(k_src + WS_TILE_BYTES, HD / 64, 0, min(WS_BN, key_lo - tile_start), lane, 32);
                __syncwarp();
            }
            warp_tile<WS_BN, 16, WS_BN>(st, q_s, 0, k_src, k_src + WS_TILE_BYTES, 0, (t0 + n) * WS_BN, hi_r, first_r, scale2);
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty0 + 8 * s) : "memory");
        }
        if (!ok && lane == 0) atomicExch(status, GAVE_UP_DECODE);
    }
    __syncthreads();

    // merge the consumer warps through shared memory (the ring is free now): rows of HD + 8 floats keep the
    // 8-byte stores of a warp's fragment off each other's banks; only the group's `rep` rows are kept
    constexpr int MS = HD + 8;
    float* sm_o = reinterpret_cast<float*>(smem);                  // [warp][16][MS]
    float* sm_ml = sm_o + WS_CONSUMERS * 16 * MS;                   // [warp][16][2]
    float* sm_f = sm_ml + WS_CONSUMERS * 16 * 2;                    // [16][WS_CONSUMERS] weights, then [16][2] (max, sum)
    float* sm_row = sm_f + 16 * WS_CONSUMERS;
    if (warp < WS_CONSUMERS) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 1);
            st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 2);
        }
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < NTO; ++n) {
            if (r0 < rep)
                *reinterpret_cast<float2*>(sm_o + (size_t)(warp * 16 + r0) * MS + n * 8 + c0) = make_float2(st.o[n][0], st.o[n][1]);
            if (r0 + 8 < rep)
                *reinterpret_cast<float2*>(sm_o + (size_t)(warp * 16 + r0 + 8) * MS + n * 8 + c0) = make_float2(st.o[n][2], st.o[n][3]);
        }
        if ((lane & 3) == 0) {
            sm_ml[(warp * 16 + r0) * 2] = st.m[0];      sm_ml[(warp * 16 + r0) * 2 + 1] = st.l[0];
            sm_ml[(warp * 16 + r0 + 8) * 2] = st.m[1];  sm_ml[(warp * 16 + r0 + 8) * 2 + 1] = st.l[1];
        }
    }
    __syncthreads();
    if ((int)threadIdx.x < rep) {            // the warps' weights exp2(m_w - M) and the row's sum, once per row
        const int row = threadIdx.x;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WS_CONSUMERS; ++w) M = fmaxf(M, sm_ml[(w * 16 + row) * 2]);
        const float mbase = M == -INFINITY ? 0.f : M;
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < WS_CONSUMERS; ++w) {
            const float f = exp2f(sm_ml[(w * 16 + row) * 2] - mbase);
            sm_f[row * WS_CONSUMERS + w] = f;
            L += sm_ml[(w * 16 + row) * 2 + 1] * f;
        }
        sm_row[row * 2] = M;
        sm_row[row * 2 + 1] = L;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rep * (HD / 4); idx += WS_THREADS) {
        const int row = idx / (HD / 4), d = (idx % (HD / 4)) * 4;
        float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < WS_CONSUMERS; ++w) {
            const float f = sm_f[row * WS_CONSUMERS + w];
            const float4 o = *reinterpret_cast<const float4*>(sm_o + (size_t)(w * 16 + row) * MS + d);
            O.x += o.x * f; O.y += o.y * f; O.z += o.z * f; O.w += o.w * f;
        }
        const int head = g * rep + row;
        if (num_splits == 1) {
            const float L = sm_row[row * 2 + 1];
            __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(out + (size_t)token * out_stride + (size_t)head * HD + d);
            dst[0] = __floats2bfloat162_rn(O.x / L, O.y / L);
            dst[1] = __floats2bfloat162_rn(O.z / L, O.w / L);
        } else {
            const size_t slot = ((size_t)r * nq + head) * max_splits + split;
            *reinterpret_cast<float4*>(part_o + slot * HD + d) = O;
            if (d == 0) { part_ml[slot * 2] = sm_row[row * 2]; part_ml[slot * 2 + 1] = sm_row[row * 2 + 1]; }
        }
    }
}

// merge of the splits: grid (nq, requests), one thread an output column.  A kernel of a few microseconds that
// stands between two others, so its own chain of dependent steps is kept short: every thread first asks for its
// column of up to 32 splits and, in the same breath, lane s of every warp for split s's maximum and sum; the
// weights exp2(m_s - M) are then worked out by every warp for itself and handed round by shuffle, so no thread
// waits for another warp and nothing passes through shared memory.  More than 32 splits are taken 32 at a
// time with a running maximum.  The sums run in split order and depend on nothing but the row.
__global__ void merge_kernel(bf16* __restrict__ out, int out_stride, const int* __restrict__ req_q_start,
                             const int* __restrict__ req_q_len, const int* __restrict__ req_ctx_len, int nq,
                             int split_keys, int max_splits, const float* __restrict__ part_o,
                             const float* __restrict__ part_ml) {
    pdl_begin();
    const int head = blockIdx.x, r = blockIdx.y;
    if (req_q_len[r] != 1) return;
    const int part_keys = keys_per_split(req_ctx_len[r], split_keys, max_splits, SPLIT_TILE);
    const int num_splits = (req_ctx_len[r] + part_keys - 1) / part_keys;
    if (num_splits <= 1) return;
    const size_t slot0 = ((size_t)r * nq + head) * max_splits;
    const int lane = threadIdx.x & 31;
    const float2* ml = reinterpret_cast<const float2*>(part_ml) + slot0;
    for (int d = threadIdx.x; d - lane < HD; d += blockDim.x) {   // a warp stays together (head sizes come in steps of 16)
        const bool live = d < HD;
        float M = -INFINITY, L = 0.f, O = 0.f;
        for (int s0 = 0; s0 < num_splits; s0 += 32) {
            float p[32];
#pragma unroll
            for (int u = 0; u < 32; ++u) p[u] = (live && s0 + u < num_splits) ? part_o[(slot0 + s0 + u) * HD + d] : 0.f;
            const float2 mine = s0 + lane < num_splits ? ml[s0 + lane] : make_float2(-INFINITY, 0.f);
            const float M_new = fmaxf(M, warp_max(mine.x));
            const float base = M_new == -INFINITY ? 0.f : M_new;
            const float keep = exp2f(M - base);                  // exp2(-inf) = 0 for the first group
            const float w = exp2f(mine.x - base);
            L = L * keep + warp_sum(mine.y * w);
            O *= keep;
#pragma unroll
            for (int u = 0; u < 32; ++u) O += p[u] * __shfl_sync(0xffffffffu, w, u);     // a split past the end has p = 0
            M = M_new;
        }
        if (live) out[(size_t)req_q_start[r] * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(O / L);
    }
}

// --------------------------------------------------------------------------------------
// prefill: grid (row tiles, nkv, requests); heavier (later) row tiles first
// --------------------------------------------------------------------------------------
constexpr int PRE_WARPS = 8;
constexpr int PRE_THREADS = PRE_WARPS * 32;
constexpr int BM = PRE_WARPS * 16;
constexpr int PRE_STAGES = 2;
constexpr int PRE_SMEM = 1024 + BM * ROWB + PRE_STAGES * 2 * TILE_BYTES + 64;

__global__ void __launch_bounds__(PRE_THREADS)
prefill_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
               const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
               const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
               const int* __restrict__ req_q_start, const int* __restrict__ req_q_len, const int* __restrict__ req_ctx_len,
               const int* __restrict__ block_table, int max_pages, int nq, int nkv, int page_size, int window, float scale2,
               int skip_single, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    pdl_begin();
    const int g = blockIdx.x, r = blockIdx.y;                 // grid (key/value heads, requests, tiles): the longest tiles start first
    const int q_len = req_q_len[r];
    if (q_len <= 0 || (skip_single && q_len == 1)) return;
    const int rep = nq / nkv, rows = q_len * rep;
    const int tile = (int)gridDim.z - 1 - (int)blockIdx.z;
    const int row0 = tile * BM;
    if (row0 >= rows) return;
    const int ctx = req_ctx_len[r], q_start = req_q_start[r], pos0 = ctx - q_len;   // position of the request's first new token
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = base + PRE_STAGES * 2 * TILE_BYTES;

    // keys this CTA needs: from the first row's window start to the last row's position
    const int last_row = min(rows, row0 + BM) - 1;
    const int pos_hi = pos0 + last_row / rep;
    const int pos_lo = pos0 + row0 / rep;
    const int key_lo = window > 0 ? max(0, pos_lo - window + 1) : 0, key_hi = pos_hi + 1;

    int pos_r[2], first_r[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = row0 + warp * 16 + (lane >> 2) + i * 8;
        pos_r[i] = m < rows ? pos0 + m / rep : -1;                      // a row past the end sees no key
        first_r[i] = window > 0 ? max(0, pos_r[i] - window + 1) : 0;
    }
    RowState st;
    init_state(st);
    TileRing<PRE_STAGES, PRE_THREADS> ring;
    ring.kv_s = base; ring.bars = q_s + BM * ROWB;
    ring.k_pages = k_pages; ring.v_pages = v_pages; ring.k_map = &k_map; ring.v_map = &v_map;
    ring.table = block_table + (size_t)r * max_pages; ring.max_pages = max_pages;
    ring.key_lo = key_lo; ring.key_hi = key_hi; ring.g = g; ring.nkv = nkv; ring.page_size = page_size;
    ring.page_shift = 31 - __clz(page_size);
    ring.t0 = key_lo / BN; ring.t1 = (key_hi + BN - 1) / BN;
    ring.ctx_end = ctx;
    ring.init();
    load_q_tile<PRE_THREADS, BM>(q_s, q, q_stride, q_start, q_len, row0, BM, g, rep);
    if (USE_TMA) cp_commit();
    ring.prologue();
    if (USE_TMA) cp_wait<0>();
    int t = ring.t0;
    bool ok = true;
    for (; t < ring.t1; ++t) {
        if (!ring.arrive(t)) { ok = false; break; }
        const int s = (t - ring.t0) % PRE_STAGES;
        // a warp whose rows all end before this tile has nothing to add
        const int warp_hi = pos0 + min(rows - 1, row0 + warp * 16 + 15) / rep;
        if (t * BN <= warp_hi && row0 + warp * 16 < rows)
            warp_tile<BN, BM>(st, q_s, warp * 16, ring.k_stage(s), ring.v_stage(s), 0, t * BN, pos_r, first_r, scale2);
    }
    ring.drain(ok ? -1 : t);
    if (!ok) {
        if (threadIdx.x == 0) atomicExch(status, GAVE_UP_PREFILL);
        return;
    }
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

#include "attention_prefill_tc.cuh"      // prefill_tc_kernel, prefill_pair_kernel (head sizes in steps of 64 / 128)

// --------------------------------------------------------------------------------------
// host side: tensor maps over the pools (cached by pointer and shape), entry points
// --------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiled encoder() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(p);
    }
    return fn;
}
struct PoolKey {
    const void* ptr; long long rows; int box_rows; bool whole_rows;
    bool operator==(const PoolKey& o) const { return ptr == o.ptr && rows == o.rows && box_rows == o.box_rows && whole_rows == o.whole_rows; }
};
struct PoolKeyHash {
    size_t operator()(const PoolKey& k) const { return std::hash<const void*>()(k.ptr) ^ (size_t)(k.rows * 31 + k.box_rows * 2 + (k.whole_rows ? 1 : 0)); }
};
static std::unordered_map<PoolKey, CUtensorMap, PoolKeyHash> g_pool_maps;
static std::mutex g_pool_mutex;

// A pool [pages][nkv][page_size][HD] as a matrix of rows x HD; boxes of box_rows x 64 columns, 128-byte swizzle.
// `whole_rows`: the columns as a third dimension of HD / 64 blocks of 64, so that one box holds whole rows and
// arrives as [block][row][64 columns], the same place that HD / 64 boxes of the flat matrix fill one by one.
static int pool_map(const void* ptr, long long rows, int box_rows, CUtensorMap* out, bool whole_rows = false) {
    if (!USE_TMA) { memset(out, 0, sizeof(*out)); return WLLM_OK; }
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    const PoolKey key{ptr, rows, box_rows, whole_rows};
    auto it = g_pool_maps.find(key);
    if (it != g_pool_maps.end()) { *out = it->second; return WLLM_OK; }
    EncodeTiled enc = encoder();
    if (!enc) return 6;
    const cuuint64_t dims[3] = {whole_rows ? 64u : (cuuint64_t)HD, (cuuint64_t)rows, (cuuint64_t)HD / 64};
    const cuuint64_t strides[2] = {(cuuint64_t)HD * 2, 128};
    const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)HD / 64};
    const cuuint32_t elem[3] = {1, 1, 1};
    CUtensorMap m;
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, whole_rows ? 3 : 2, const_cast<void*>(ptr), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 2000 + (int)r;
    if (g_pool_maps.size() > 4096) g_pool_maps.clear();
    g_pool_maps[key] = m;
    *out = m;
    return WLLM_OK;
}

WLLM_API int wllm_attention_mma_head_dim() { return HD; }

// Arrival counters of the prefill tiles that two CTAs share; zero between launches (the merging CTA resets
// its counter).  One set per device: launches that may overlap in time (two streams) must not share it, and
// the engine has one stream.
constexpr int ARRIVAL_SLOTS = 1 << 16;
static __device__ int g_tile_arrivals[ARRIVAL_SLOTS];
template <typename Symbol>
static int* symbol_address(const Symbol& symbol, int** cache) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (cache[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, symbol) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        cache[dev] = static_cast<int*>(p);
    }
    return cache[dev];
}
static int* tile_arrivals_address() {
    static int* addr[64];
    return symbol_address(g_tile_arrivals, addr);
}

// Floats of scratch the decode path needs for `requests` requests: partial outputs and (max, sum) pairs.
WLLM_API long long wllm_attention_mma_scratch_floats(int requests, int nq, int max_splits) {
    return (long long)requests * nq * max_splits * (HD + 2);
}

static int check_common(const void* q, int q_stride, const void* out, int out_stride, const void* k_pages,
                        const void* v_pages, int nq, int nkv, int page_size, long long pool_pages) {
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size < 16 || (page_size & (page_size - 1)) || pool_pages < 1)
        return WLLM_BAD_SIZE;
    if (q_stride % 8 != 0 || out_stride % 2 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)out & 3) ||
        ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
        return WLLM_BAD_ALIGN;
    return WLLM_OK;
}

// Tokens of requests with q_len == 1.  `scratch` holds wllm_attention_mma_scratch_floats(...) floats;
// `pool_pages` is the number of pages of k_pages / v_pages; `status` is a device int that stays 0 unless
// a CTA gave up waiting for a tile.
WLLM_API int wllm_attention_mma_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                       const void* v_pages, long long pool_pages, const int* req_q_start,
                                       const int* req_q_len, const int* req_ctx_len, const int* block_table,
                                       int max_pages, int requests, int nq, int nkv, int page_size, int window,
                                       float scale, int split_keys, int max_splits, float* scratch, int* status,
                                       cudaStream_t stream) {
    if (requests <= 0) return WLLM_OK;
    const int bad = check_common(q, q_stride, out, out_stride, k_pages, v_pages, nq, nkv, page_size, pool_pages);
    if (bad) return bad;
    const int tile = USE_TMA ? WS_BN : BN;      // splits are whole tiles of the kernel that runs
    if (nq / nkv > 16 || split_keys < BN || split_keys % tile != 0 || max_splits < 1 || max_splits > MERGE_MAX_SPLITS ||
        nkv > 65535)
        return WLLM_BAD_SIZE;
    CUtensorMap km, vm;
    const long long rows = pool_pages * nkv * page_size;
    const int box_rows = USE_TMA ? (page_size < WS_BN ? page_size : WS_BN) : (page_size < BN ? page_size : BN);
    const bool whole_rows = USE_TMA && box_rows == WS_BN;      // pages of at least a tile's keys: one copy a tile
    int r = pool_map(k_pages, rows, box_rows, &km, whole_rows);
    if (r) return r;
    r = pool_map(v_pages, rows, box_rows, &vm, whole_rows);
    if (r) return r;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = USE_TMA
            ? cudaFuncSetAttribute(decode_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WS_SMEM)
            : cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        configured = true;
    }
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)requests * nq * max_splits * HD;
    if ((long long)requests * nkv * max_splits <= 148) split_keys = -split_keys;     // resident at once: cut evenly
    int st;
    if (USE_TMA)
        st = wllm_launch(decode_ws_kernel, dim3(requests, nkv, max_splits), WS_THREADS, WS_SMEM, stream,
                         (const bf16*)q, q_stride, (bf16*)out, out_stride, km, vm, req_q_start, req_q_len, req_ctx_len,
                         block_table, max_pages, nq, nkv, page_size, window, scale * LOG2E, split_keys, max_splits, part_o,
                         part_ml, whole_rows ? 1 : 0, status);
    else
        st = wllm_launch(decode_kernel, dim3(requests, nkv, max_splits), NTHREADS, DEC_SMEM, stream,
                         (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_pages, (const bf16*)v_pages, km, vm,
                         req_q_start, req_q_len, req_ctx_len, block_table, max_pages, nq, nkv, page_size, window,
                         scale * LOG2E, split_keys, max_splits, part_o, part_ml, status);
    if (st || max_splits == 1) return st;
    return wllm_launch(merge_kernel, dim3(nq, requests), HD >= 256 ? 256 : (HD >= 128 ? 128 : 64), 0, stream,
                       (bf16*)out, out_stride, req_q_start, req_q_len, req_ctx_len, nq, split_keys, max_splits,
                       (const float*)part_o, (const float*)part_ml);
}

// Floats of `halves` for a prefill launch that shares tiles between two CTAs.
WLLM_API long long wllm_attention_mma_prefill_halves_floats(int requests, int max_q_len, int nq, int nkv) {
    const long long tiles = ((long long)max_q_len * (nq / nkv) + 127) / 128;
    return tiles * nkv * requests * 2 * 128 * (HD + 4);
}

// Tokens of requests with q_len > 1 (and of those with q_len == 1 too unless skip_single).
WLLM_API int wllm_attention_mma_prefill(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                        const void* v_pages, long long pool_pages, const int* req_q_start,
                                        const int* req_q_len, const int* req_ctx_len, const int* block_table,
                                        int max_pages, int requests, int max_q_len, int nq, int nkv, int page_size,
                                        int window, float scale, int skip_single, int split_above, float* halves,
                                        int* status, cudaStream_t stream) {
    // split_above > 0 (tensor-memory kernel only): a tile of 128 rows that walks more than split_above tiles of
    // 64 keys is shared by two CTAs; `halves` then holds wllm_attention_mma_prefill_halves_floats(...) floats.
    if (requests <= 0 || max_q_len <= 0) return WLLM_OK;
    const int bad = check_common(q, q_stride, out, out_stride, k_pages, v_pages, nq, nkv, page_size, pool_pages);
    if (bad) return bad;
    CUtensorMap km, vm;
    const long long rows = pool_pages * nkv * page_size;
    int r = pool_map(k_pages, rows, page_size < BN ? page_size : BN, &km);
    if (r) return r;
    r = pool_map(v_pages, rows, page_size < BN ? page_size : BN, &vm);
    if (r) return r;
    static bool configured = false;
#if (HEAD_DIM % 64 == 0)
    static bool use_tc = false;
#endif
#if (HEAD_DIM % 128 == 0)
    static bool use_pair = false;
#endif
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PRE_SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
#if (HEAD_DIM % 64 == 0)
        e = cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        const char* legacy = getenv("WLLM_ATTENTION_MMA");       // =1: the mma.sync kernel, for comparison
        use_tc = !(legacy && legacy[0] == '1');
#endif
#if (HEAD_DIM % 128 == 0)
        e = cudaFuncSetAttribute(prefill_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PR_SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        const char* single = getenv("WLLM_ATTENTION_PAIR");      // =0: one CTA a tile always
        use_pair = !(single && single[0] == '0');
#endif
        configured = true;
    }
    const int tiles = (max_q_len * (nq / nkv) + BM - 1) / BM;
    if (requests > 65535 || 2LL * tiles > 65535) return WLLM_BAD_SIZE;      // the grid's y and z
#if (HEAD_DIM % 64 == 0)
#if (HEAD_DIM % 128 == 0)
    // more than one tile of 128 rows in the longest request: pairs of CTAs on 256-row tiles
    if (use_tc && use_pair && max_q_len * (nq / nkv) > TC_BM && (out_stride % 8 == 0) && (((uintptr_t)out & 15) == 0)) {
        const int pair_tiles = (max_q_len * (nq / nkv) + 2 * TC_BM - 1) / (2 * TC_BM);
        return wllm_launch(prefill_pair_kernel, dim3(2 * nkv, requests, pair_tiles), TC_THREADS, PR_SMEM, stream,
                           (const bf16*)q, q_stride, (bf16*)out, out_stride, km, vm, req_q_start, req_q_len, req_ctx_len,
                           block_table, max_pages, nq, nkv, page_size, window, scale * LOG2E, skip_single, status);
    }
#endif
    if (use_tc && (out_stride % 8 == 0) && (((uintptr_t)out & 15) == 0)) {
        int* arrivals = nullptr;
        if (split_above > 0) {
            if (halves == nullptr || ((uintptr_t)halves & 15) || (long long)tiles * nkv * requests > ARRIVAL_SLOTS) return WLLM_BAD_SIZE;
            arrivals = tile_arrivals_address();
            if (arrivals == nullptr) split_above = 0;
        }
        return wllm_launch(prefill_tc_kernel, dim3(nkv, requests, split_above > 0 ? 2 * tiles : tiles), TC_THREADS, TC_SMEM, stream,
                           (const bf16*)q, q_stride, (bf16*)out, out_stride, km, vm, req_q_start, req_q_len, req_ctx_len,
                           block_table, max_pages, nq, nkv, page_size, window, scale * LOG2E, skip_single, split_above, halves,
                           arrivals, status);
    }
#endif
    return wllm_launch(prefill_kernel, dim3(nkv, requests, tiles), PRE_THREADS, PRE_SMEM, stream,
                       (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_pages, (const bf16*)v_pages, km, vm,
                       req_q_start, req_q_len, req_ctx_len, block_table, max_pages, nq, nkv, page_size, window, scale * LOG2E,
                       skip_single, status);
}
