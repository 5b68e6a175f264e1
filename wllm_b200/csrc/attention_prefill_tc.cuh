// The prefill attention kernels on the fifth-generation tensor cores (tcgen05, tensor memory, TMA): one CTA a
// tile of 128 query rows for head sizes in steps of 64, and pairs of CTAs on 256-row tiles for head sizes in
// steps of 128.  Included by attention_mma.cu, whose constants (HD, ROWB, CPR), swizzle and copy helpers and
// status codes it uses; compiled per head size like the rest of that file.
#pragma once
#if (HEAD_DIM % 64 == 0)
// --------------------------------------------------------------------------------------
// prefill on the fifth-generation tensor cores (head sizes in steps of 64): grid as above
// --------------------------------------------------------------------------------------
// 128 query rows per CTA are the 128 lanes of tensor memory.  Shared memory holds nothing but key and value
// tiles: the kernel is bound by shared-memory bandwidth when the tensor core has to read Q (for the scores)
// and P (for the output) from there beside K and V, so both A operands live in tensor memory instead.
// Columns: O [0, head size), two score buffers of 64 at 256 and 320, Q (two elements a column) from 384.
// Roles by warp:
//   warps 0, 6  one lane of warp 0 issues the TMA box copies of the key tiles, one lane of warp 6 those of
//               the value tiles (64 keys each, three stages each, on barriers of their own: a key stage is
//               free as soon as its scores are computed, a value stage once it has been accumulated);
//   warp 1      one lane issues tcgen05.mma: scores S = Q K^T (M 128, N 64, K = head size; Q from tensor
//               memory) into one of two score buffers, one tile ahead of the softmax, and O += P V (M 128,
//               N = head size, K 64) with P from tensor memory and V as an MN-major operand straight from
//               the value tile (no transpose);
//   warps 2-5   one thread per row: store the row of Q into tensor memory once; then per tile read the
//               row's 64 scores with tcgen05.ld, mask, scale, running maximum and sum in registers without
//               a shuffle, write P as bfloat16 over the scores it has just read, and rescale the row of O
//               only when some row of the warp has a new maximum.  At the end they normalise O and store it.
// The tensor core runs its instructions in the order of issue: S(n + 2) is issued after P V(n), which reads
// the P that lies in S(n + 2)'s buffer, so the buffers need no barrier of their own.
// All waits are bounded; a role that gives up records a code and every role leaves through the common
// exit, where tensor memory is freed.
constexpr int TC_BM = 128, TC_BN = 64, TC_KV_STAGES = 3;
constexpr int TC_KV_BYTES = TC_BN * ROWB;
constexpr int TC_SMEM = 1024 + 2 * TC_KV_STAGES * TC_KV_BYTES + 256;
constexpr int TC_THREADS = 224;
constexpr int TC_S_COL = 256;                      // score buffers behind the output accumulator
constexpr int TC_Q_COL = 384;                      // the query tile: HD / 2 columns
constexpr float TC_MAX_SLACK = 8.0f;
constexpr uint32_t IDESC_S = umma_idesc(TC_BM, TC_BN, false, false);
constexpr uint32_t IDESC_PV = umma_idesc(TC_BM, HD, false, true);       // V is MN-major
enum { GAVE_UP_TC_LOAD = 23, GAVE_UP_TC_MMA = 24, GAVE_UP_TC_SOFTMAX = 25 };

__device__ __forceinline__ float fast_exp2(float x) {       // ex2.approx: 2 ulp, exp2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(TC_THREADS, 1)
prefill_tc_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                  const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                  const int* __restrict__ req_q_start, const int* __restrict__ req_q_len, const int* __restrict__ req_ctx_len,
                  const int* __restrict__ block_table, int max_pages, int nq, int nkv, int page_size, int window, float scale2,
                  int skip_single, int split_above, float* __restrict__ halves, int* __restrict__ arrivals,
                  int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ int s_second;
    pdl_begin();
    // grid (key/value heads, requests, tiles): CTAs start in the order x, y, z, so the tiles that walk the most
    // keys (the last rows of every head and request) start first and the short ones fill the SMs behind them
    const int g = blockIdx.x, r = blockIdx.y;
    const int q_len = req_q_len[r];
    if (q_len <= 0 || (skip_single && q_len == 1)) return;
    const int rep = nq / nkv, rows = q_len * rep;
    // With split_above > 0 the grid holds two CTAs a tile; a tile that walks more than split_above key tiles
    // is shared between them (each takes half of its keys), the second CTA of any other tile leaves at once.
    const int parts = split_above > 0 ? 2 : 1;
    const int slot_x = (int)gridDim.z - 1 - (int)blockIdx.z;
    const int tile = slot_x / parts, part = slot_x % parts;
    const int row0 = tile * TC_BM;
    if (row0 >= rows) return;
    const int ctx = req_ctx_len[r], q_start = req_q_start[r], pos0 = ctx - q_len;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t k_s = base, v_s = k_s + TC_KV_STAGES * TC_KV_BYTES, bars = v_s + TC_KV_STAGES * TC_KV_BYTES;
    const uint32_t k_full = bars, k_empty = k_full + 8 * TC_KV_STAGES, v_full = k_empty + 8 * TC_KV_STAGES;
    const uint32_t v_empty = v_full + 8 * TC_KV_STAGES, s_full = v_empty + 8 * TC_KV_STAGES;
    const uint32_t q_full = s_full + 16, p_full = q_full + 8, pv_done = p_full + 8, tmem_slot = pv_done + 8;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int last_row = min(rows, row0 + TC_BM) - 1;
    const int pos_hi = pos0 + last_row / rep, pos_lo = pos0 + row0 / rep;
    const int key_lo = window > 0 ? max(0, pos_lo - window + 1) : 0, key_hi = pos_hi + 1;
    int t0 = key_lo / TC_BN, t1 = (key_hi + TC_BN - 1) / TC_BN, T = t1 - t0;
    const bool shared_tile = split_above > 0 && T > split_above;
    if (!shared_tile && part == 1) return;
    if (shared_tile) {          // both halves hold keys of every row: a tile spans at most two key tiles of positions
        const int mid = t0 + (T + 1) / 2;
        if (part == 0) t1 = mid; else t0 = mid;
        T = t1 - t0;
    }
    const int page_shift = 31 - __clz(page_size);
    const int* table = block_table + (size_t)r * max_pages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_KV_STAGES; ++s) {
            mbar_init(k_full + 8 * s, 1); mbar_init(k_empty + 8 * s, 1);
            mbar_init(v_full + 8 * s, 1); mbar_init(v_empty + 8 * s, 1);
        }
        mbar_init(s_full, 1); mbar_init(s_full + 8, 1);
        mbar_init(q_full, 4);
        mbar_init(p_full, 4);
        mbar_init(pv_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tc_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0 || warp == 6) {
        // ---------------- TMA producers: warp 0 the key tiles, warp 6 the value tiles ----------------
        // (one thread for both would hold back the next key tile while it waits for a value stage, which
        // is handed back a tile later than the key stage of the same tile)
        if (lane == 0) {
            const int kv = warp == 6;
            const uint32_t full0 = kv ? v_full : k_full, empty0 = kv ? v_empty : k_empty, ring = kv ? v_s : k_s;
            const CUtensorMap* map = kv ? &v_map : &k_map;
            const int box_rows = page_size < TC_BN ? page_size : TC_BN;
            bool ok = true;
            int n = 0;
            for (; n < T && ok; ++n) {
                const int s = n % TC_KV_STAGES, ph = (n / TC_KV_STAGES) & 1, tile_start = (t0 + n) * TC_BN;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) { ok = false; break; }
                const uint32_t bar = full0 + 8 * s, dst = ring + s * TC_KV_BYTES;
                mbar_expect_tx(bar, TC_KV_BYTES);
                for (int r0 = 0; r0 < TC_BN; r0 += box_rows) {
                    const int key = tile_start + r0, index = key >> page_shift;
                    int page = index < max_pages ? table[index] : 0;
                    if (page < 0) page = 0;
                    const int row = (page * nkv + g) * page_size + (key & (page_size - 1));
#pragma unroll
                    for (int cb = 0; cb < HD / 64; ++cb)
                        tma_load_2d(dst + cb * (TC_BN * 128) + r0 * 128, map, bar, cb * 64, row);
                }
            }
            // stay until the stages that were filled have been handed back: nothing in flight at the exit
            for (int k = 0; k < TC_KV_STAGES && ok; ++k, ++n) {
                const int s = n % TC_KV_STAGES, ph = (n / TC_KV_STAGES) & 1;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) ok = false;
            }
            if (!ok) atomicExch(status, GAVE_UP_TC_LOAD);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            bool ok = mbar_wait(q_full, 0);
            tc_fence_after();
            auto issue_scores = [&](int n) -> bool {       // S(n) = Q K(n)^T into score buffer n % 2
                const int s = n % TC_KV_STAGES, ph = (n / TC_KV_STAGES) & 1;
                if (!mbar_wait(k_full + 8 * s, ph)) return false;
                tc_fence_after();
                const uint32_t d = tmem_base + TC_S_COL + (n & 1) * TC_BN, kb = k_s + s * TC_KV_BYTES;
#pragma unroll
                for (int kt = 0; kt < HD / 16; ++kt)
                    tc_mma_ts(d, tmem_base + TC_Q_COL + kt * 8, smem_desc(kb + (kt >> 2) * (TC_BN * 128) + (kt & 3) * 32),
                              IDESC_S, kt > 0 ? 1u : 0u);
                tc_commit(k_empty + 8 * s);
                tc_commit(s_full + 8 * (n & 1));
                return true;
            };
            ok = ok && issue_scores(0);
            for (int n = 0; n < T && ok; ++n) {
                if (n + 1 < T && !issue_scores(n + 1)) { ok = false; break; }
                const int s = n % TC_KV_STAGES, ph = (n / TC_KV_STAGES) & 1;
                if (!mbar_wait(v_full + 8 * s, ph) || !mbar_wait(p_full, n & 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t vb = v_s + s * TC_KV_BYTES, pa = tmem_base + TC_S_COL + (n & 1) * TC_BN;
#pragma unroll
                for (int kk = 0; kk < TC_BN / 16; ++kk)
                    tc_mma_ts(tmem_base, pa + kk * 8, smem_desc_mn(vb + kk * (16 * 128), TC_BN * 128), IDESC_PV,
                              (n > 0 || kk > 0) ? 1u : 0u);
                tc_commit(v_empty + 8 * s);
                tc_commit(pv_done);
            }
            if (!ok) atomicExch(status, GAVE_UP_TC_MMA);
        }
    } else {
        // ---------------- softmax: one thread per row ----------------
        const int quarter = warp & 3, row = quarter * 32 + lane, m_row = row0 + row;
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        // the row of Q into tensor memory: element pairs (k, k + 1) share a column
        {
            const bf16* src = m_row < rows ? q + (size_t)(q_start + m_row / rep) * q_stride + (size_t)(g * rep + m_row % rep) * HD : nullptr;
            constexpr int QC = (HD / 2) % 64 == 0 ? 64 : 32;       // columns a round: sixteen (or eight) loads in flight
#pragma unroll 1
            for (int c0 = 0; c0 < HD / 2; c0 += QC) {
                uint32_t w[QC / 32][32];
#pragma unroll
                for (int j = 0; j < QC / 4; ++j) {
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (src) v = *reinterpret_cast<const uint4*>(src + 2 * c0 + 8 * j);
                    w[j / 8][4 * (j % 8)] = v.x; w[j / 8][4 * (j % 8) + 1] = v.y;
                    w[j / 8][4 * (j % 8) + 2] = v.z; w[j / 8][4 * (j % 8) + 3] = v.w;
                }
#pragma unroll
                for (int h = 0; h < QC / 32; ++h) tc_st32(t_lane + TC_Q_COL + c0 + 32 * h, w[h]);
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full);
        }

        const int pos_row = m_row < rows ? pos0 + m_row / rep : -1;            // a row past the end sees no key
        const int first_row = window > 0 ? max(0, pos_row - window + 1) : 0;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int n = 0; n < T; ++n) {
            const int b = n & 1, ph = (n >> 1) & 1, key0 = (t0 + n) * TC_BN;
            if (!mbar_wait(s_full + 8 * b, ph)) { ok = false; break; }
            tc_fence_after();
            uint32_t sv[2][32];
            tc_ld32(t_lane + TC_S_COL + b * TC_BN, sv[0]);
            tc_ld32(t_lane + TC_S_COL + b * TC_BN + 32, sv[1]);
            tc_wait_ld();
            // Scores stay unscaled until the exponent: max(scale * s) = scale * max(s) for scale > 0, and
            // exp2(scale * s - scale * m) is one fused multiply-add and one ex2 per element.  Only tiles at the
            // causal edge or the window's start need the per-key mask; the warp decides together.
            const bool inner = __all_sync(0xffffffffu, key0 + TC_BN - 1 <= pos_row && key0 >= first_row);
            // One warp runs alone on its scheduler, so a chain of dependent maxima or additions would cost its
            // full latency per element: four independent chains each (the order is fixed all the same).
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (inner) {
#pragma unroll
                for (int c = 0; c < 64; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sv[c >> 5][c & 31]));
            } else {
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const int key = key0 + c;
                    const float v = (key <= pos_row && key >= first_row) ? __uint_as_float(sv[c >> 5][c & 31]) : -INFINITY;
                    sv[c >> 5][c & 31] = __float_as_uint(v);
                    mx4[c & 3] = fmaxf(mx4[c & 3], v);
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // The reference point of the exponents follows the running maximum lazily: it moves only when the
            // maximum has grown by more than TC_MAX_SLACK (in units of log2), so the probabilities stay below
            // 2^slack and the row of O has to be rescaled in few tiles instead of in most.  The quotient O / l
            // does not depend on the reference point.
            const float m_tile = fmaxf(m_run, mx * scale2);
            const float m_new = m_tile > m_run + TC_MAX_SLACK ? m_tile : m_run;      // m_run = -inf: takes m_tile
            const float mbase = m_new == -INFINITY ? 0.f : m_new;
            const float corr = fast_exp2(m_run - mbase);
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t packed[32];
#pragma unroll
            for (int c = 0; c < 64; c += 2) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(sv[c >> 5][c & 31]), scale2, -mbase));
                const float p1 = fast_exp2(fmaf(__uint_as_float(sv[(c + 1) >> 5][(c + 1) & 31]), scale2, -mbase));
                sum4[(c >> 1) & 3] += p0 + p1;
                packed[c >> 1] = pack_bf16(p0, p1);
            }
            l_run = l_run * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            const bool changed = m_new > m_run;
            m_run = m_new;
            // P over the scores this thread has just read: keys (2j, 2j + 1) in column j of the buffer
            tc_st32(t_lane + TC_S_COL + b * TC_BN, packed);
            if (key0 + TC_BN > ctx || key0 < key_lo) {
                // The value tile reaches past the request's last key (or in front of the window's first): those rows
                // hold whatever the page holds, and a weight of zero times something that is no number is no zero.
                // They are cleared before this warp reports P, which is what the output product waits for.
                const int vs = n % TC_KV_STAGES;
                if (!mbar_wait(v_full + 8 * vs, (n / TC_KV_STAGES) & 1)) { ok = false; break; }
                const uint32_t vt = v_s + vs * TC_KV_BYTES;
                if (key0 + TC_BN > ctx) zero_value_rows<TC_BN>(vt, HD / 64, max(0, ctx - key0), TC_BN, threadIdx.x - 64, 128);
                if (key0 < key_lo) zero_value_rows<TC_BN>(vt, HD / 64, 0, min(TC_BN, key_lo - key0), threadIdx.x - 64, 128);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            if (n > 0) {
                if (!mbar_wait(pv_done, (n - 1) & 1)) { ok = false; break; }     // O of the tile before is complete
                tc_fence_after();
                if (__any_sync(0xffffffffu, changed)) {
#pragma unroll 1
                    for (int c0 = 0; c0 < HD; c0 += 32) {
                        uint32_t ov[32];
                        tc_ld32(t_lane + c0, ov);
                        tc_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * corr);
                        tc_st32(t_lane + c0, ov);
                    }
                }
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        if (ok && !mbar_wait(pv_done, (T - 1) & 1)) ok = false;
        ok = __all_sync(0xffffffffu, ok);        // the tensor-memory loads below are collective: all lanes or none
        bf16* dst = m_row < rows ? out + (size_t)(q_start + m_row / rep) * out_stride + (size_t)(g * rep + m_row % rep) * HD : nullptr;
        if (shared_tile) {
            // Two CTAs hold halves of this tile's keys.  Each writes its half result (unnormalised O, reference
            // maximum, sum) and counts itself in; the one that comes second adds the other's to its own, which
            // is still in tensor memory.  Products and sums are written so that the result does not depend
            // on which of the two that is (a * fa + b * fb with separate roundings is symmetric).
            // (every softmax thread passes the two block barriers below, whatever its own waits came to)
            // Every lane of a warp takes part in the loads, rows past the end too; only their stores are left out.
            tc_fence_after();
            const int item = (r * nkv + g) * ((int)gridDim.z / 2) + tile;
            // a half result: [column chunk of 32][row][32] (a warp writes whole lines), then (maximum, sum) by row
            float* mine = halves + (size_t)(item * 2 + part) * TC_BM * (HD + 4);
            const float* other = halves + (size_t)(item * 2 + (part ^ 1)) * TC_BM * (HD + 4);
#pragma unroll 1
            for (int c0 = 0; c0 < HD && ok; c0 += 32) {
                uint32_t ov[32];
                tc_ld32(t_lane + c0, ov);
                tc_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; c += 4)
                    *reinterpret_cast<float4*>(mine + ((size_t)c0 * TC_BM + row * 32) + c) = make_float4(__uint_as_float(ov[c]), __uint_as_float(ov[c + 1]),
                                                                            __uint_as_float(ov[c + 2]), __uint_as_float(ov[c + 3]));
            }
            mine[(size_t)HD * TC_BM + row * 2] = m_run;
            mine[(size_t)HD * TC_BM + row * 2 + 1] = l_run;
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (row == 0) {
                const int before = atomicAdd(&arrivals[item], 1);
                s_second = before;
                if (before == 1) arrivals[item] = 0;            // ready for the next launch
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (s_second == 1 && ok) {
                __threadfence();
                const float m_b = __ldcg(other + (size_t)HD * TC_BM + row * 2), l_b = __ldcg(other + (size_t)HD * TC_BM + row * 2 + 1);
                const float M = fmaxf(m_run, m_b), mb = M == -INFINITY ? 0.f : M;
                const float fa = exp2f(m_run - mb), fb = exp2f(m_b - mb);
                const float inv = 1.0f / __fadd_rn(__fmul_rn(l_run, fa), __fmul_rn(l_b, fb));
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t ov[32];
                    tc_ld32(t_lane + c0, ov);
                    tc_wait_ld();
                    float y[32];
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        const float4 b = __ldcg(reinterpret_cast<const float4*>(other + ((size_t)c0 * TC_BM + row * 32) + c));
                        y[c] = __fadd_rn(__fmul_rn(__uint_as_float(ov[c]), fa), __fmul_rn(b.x, fb)) * inv;
                        y[c + 1] = __fadd_rn(__fmul_rn(__uint_as_float(ov[c + 1]), fa), __fmul_rn(b.y, fb)) * inv;
                        y[c + 2] = __fadd_rn(__fmul_rn(__uint_as_float(ov[c + 2]), fa), __fmul_rn(b.z, fb)) * inv;
                        y[c + 3] = __fadd_rn(__fmul_rn(__uint_as_float(ov[c + 3]), fa), __fmul_rn(b.w, fb)) * inv;
                    }
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 o;
                        o.x = pack_bf16(y[c], y[c + 1]); o.y = pack_bf16(y[c + 2], y[c + 3]);
                        o.z = pack_bf16(y[c + 4], y[c + 5]); o.w = pack_bf16(y[c + 6], y[c + 7]);
                        if (dst) *reinterpret_cast<uint4*>(dst + c0 + c) = o;
                    }
                }
            }
            if (!ok && lane == 0) atomicExch(status, GAVE_UP_TC_SOFTMAX);
        } else if (ok) {
            tc_fence_after();
            const float inv = 1.0f / l_run;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t ov[32];
                tc_ld32(t_lane + c0, ov);
                tc_wait_ld();
                if (dst) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 o;
                        o.x = pack_bf16(__uint_as_float(ov[c]) * inv, __uint_as_float(ov[c + 1]) * inv);
                        o.y = pack_bf16(__uint_as_float(ov[c + 2]) * inv, __uint_as_float(ov[c + 3]) * inv);
                        o.z = pack_bf16(__uint_as_float(ov[c + 4]) * inv, __uint_as_float(ov[c + 5]) * inv);
                        o.w = pack_bf16(__uint_as_float(ov[c + 6]) * inv, __uint_as_float(ov[c + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + c) = o;
                    }
                }
            }
        } else if (lane == 0) {
            atomicExch(status, GAVE_UP_TC_SOFTMAX);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tc_dealloc(tmem_base, 512);
    }
}

#if (HEAD_DIM % 128 == 0)
// --------------------------------------------------------------------------------------
// prefill on pairs of CTAs: 256 query rows a tile, score tiles of 128 keys
// (head sizes in steps of 128: each CTA holds half of the head's columns of V in whole 64-column blocks)
// --------------------------------------------------------------------------------------
// The tensor core takes an instruction of N = 64 no faster than one of N = 128, so the sixteen score products
// of a 64-key tile cost the kernel above as much as its output products.  Score tiles of 128 keys need a
// second 128-column score buffer, which tensor memory has beside a 256-column O only when Q moves back to
// shared memory, and shared memory has room for Q and 128-key stages only when two CTAs share the keys and
// values: a cluster of two CTAs takes 256 query rows (128 each, with its own Q, O, scores and softmax), and
// tcgen05.mma.cta_group::2, issued by the first CTA for both, reads half of every operand B from each:
//   S = Q K^T   M 256, N 128 keys, K = head size; each CTA holds 64 of the 128 keys of a stage;
//   O += P V    M 256, N = head size, K 128 keys; P from tensor memory (over the scores it came from),
//               V MN-major, each CTA holding half of the head's columns for all 128 keys.
// Barriers as in the two-CTA GEMM: `full` barriers (and q_full, p_full) live in the first CTA and are
// arrived on by both; `empty`, s_full and pv_done exist in both and are arrived on by commit multicast.
// Both CTAs allocate and free tensor memory together and pass a cluster barrier before they leave.
constexpr int PR_BN = 128, PR_STAGES = 2;
constexpr int PR_Q_BYTES = TC_BM * ROWB;                   // this CTA's 128 query rows
constexpr int PR_K_BYTES = (PR_BN / 2) * ROWB;             // 64 keys x head size
constexpr int PR_V_BYTES = PR_BN * (ROWB / 2);             // 128 keys x half the head size
constexpr int PR_SMEM = 1024 + PR_Q_BYTES + PR_STAGES * (PR_K_BYTES + PR_V_BYTES) + 256;
constexpr uint32_t IDESC_PR_S = umma_idesc(2 * TC_BM, PR_BN, false, false);
constexpr uint32_t IDESC_PR_PV = umma_idesc(2 * TC_BM, HD, false, true);

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
prefill_pair_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                    const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                    const int* __restrict__ req_q_start, const int* __restrict__ req_q_len, const int* __restrict__ req_ctx_len,
                    const int* __restrict__ block_table, int max_pages, int nq, int nkv, int page_size, int window, float scale2,
                    int skip_single, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    pdl_begin();
    // grid (2 x key/value heads, requests, tiles): the pairs start in the order x, y, z, the tiles that walk the most
    // keys (the last rows of every head and request) first, so that the short ones fill the SMs behind them
    const int g = blockIdx.x >> 1, r = blockIdx.y;
    const int q_len = req_q_len[r];
    if (q_len <= 0 || (skip_single && q_len == 1)) return;             // the same for both CTAs of a pair
    const int rep = nq / nkv, rows = q_len * rep;
    const uint32_t rank = cluster_ctarank();
    const int tile = (int)gridDim.z - 1 - (int)blockIdx.z;
    if (tile * 2 * TC_BM >= rows) return;
    const int row0 = tile * 2 * TC_BM + (int)rank * TC_BM;             // may lie past the end: then all rows are masked
    const int ctx = req_ctx_len[r], q_start = req_q_start[r], pos0 = ctx - q_len;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = base, k_s = q_s + PR_Q_BYTES, v_s = k_s + PR_STAGES * PR_K_BYTES;
    const uint32_t bars = v_s + PR_STAGES * PR_V_BYTES;
    const uint32_t k_full = bars, k_empty = k_full + 8 * PR_STAGES, v_full = k_empty + 8 * PR_STAGES;
    const uint32_t v_empty = v_full + 8 * PR_STAGES, s_full = v_empty + 8 * PR_STAGES;
    const uint32_t q_full = s_full + 16, p_full = q_full + 8, pv_done = p_full + 8, tmem_slot = pv_done + 8;
    const uint32_t v_edge = tmem_slot + 8;          // this CTA's own: the value tiles that need clearing land on it
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    // the keys that the pair's 256 rows see
    const int last_row = min(rows, (tile + 1) * 2 * TC_BM) - 1;
    const int pos_hi = pos0 + last_row / rep, pos_lo = pos0 + (tile * 2 * TC_BM) / rep;
    const int key_lo = window > 0 ? max(0, pos_lo - window + 1) : 0, key_hi = pos_hi + 1;
    const int t0 = key_lo / PR_BN, t1 = (key_hi + PR_BN - 1) / PR_BN, T = t1 - t0;
    const int page_shift = 31 - __clz(page_size);
    const int* table = block_table + (size_t)r * max_pages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PR_STAGES; ++s) {
            mbar_init(k_full + 8 * s, 2); mbar_init(k_empty + 8 * s, 1);
            mbar_init(v_full + 8 * s, 2); mbar_init(v_empty + 8 * s, 1);
        }
        mbar_init(s_full, 1); mbar_init(s_full + 8, 1);
        mbar_init(q_full, 8);
        mbar_init(p_full, 8);
        mbar_init(pv_done, 1);
        mbar_init(v_edge, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tc_alloc_pair(tmem_slot, 512);
    tc_fence_before();
    cluster_sync();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    const uint32_t lead_k_full = cluster_map(k_full, 0), lead_v_full = cluster_map(v_full, 0);
    const uint32_t lead_q_full = cluster_map(q_full, 0), lead_p_full = cluster_map(p_full, 0);

    if (warp == 0 || warp == 6) {
        // ---------------- TMA producers: warp 0 this CTA's half of the key tiles, warp 6 of the value tiles ----------------
        if (lane == 0) {
            const int kv = warp == 6;
            const uint32_t full0 = kv ? lead_v_full : lead_k_full, empty0 = kv ? v_empty : k_empty;
            const uint32_t ring = kv ? v_s : k_s, stage_bytes = kv ? PR_V_BYTES : PR_K_BYTES;
            const CUtensorMap* map = kv ? &v_map : &k_map;
            const int box_rows = page_size < 64 ? page_size : 64;
            // keys: rows [64 * rank, +64) of the tile, all columns; values: all 128 rows, columns [HD/2 * rank, +HD/2)
            const int row_lo = kv ? 0 : 64 * (int)rank, row_n = kv ? PR_BN : 64;
            const int col_lo = kv ? (HD / 2) * (int)rank : 0, col_blocks = kv ? HD / 128 : HD / 64;
            bool ok = true;
            int n = 0, edges = 0;
            for (; n < T && ok; ++n) {
                const int s = n % PR_STAGES, ph = (n / PR_STAGES) & 1, tile_start = (t0 + n) * PR_BN + row_lo;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) { ok = false; break; }
                const uint32_t bar = full0 + 8 * s, dst = ring + s * stage_bytes;
                // A value tile that reaches past the request's last key (or in front of the window's first) holds, in
                // those rows, whatever the page holds; their weight is zero, but zero times something that is no
                // number is no zero.  Such a tile (the last of a request's last rows) lands on a barrier of this CTA's
                // own, its stray rows are cleared, and only then is it announced on the pair's barrier, by a plain
                // arrival in place of the byte count.
                const int key0 = (t0 + n) * PR_BN;
                const bool edge = kv && (key0 + PR_BN > ctx || key0 < key_lo);
                if (edge) mbar_expect_tx(v_edge, stage_bytes); else mbar_expect_tx_cluster(bar, stage_bytes);
                for (int r0 = 0; r0 < row_n; r0 += box_rows) {
                    const int key = tile_start + r0, index = key >> page_shift;
                    int page = index < max_pages ? table[index] : 0;
                    if (page < 0) page = 0;
                    const int row = (page * nkv + g) * page_size + (key & (page_size - 1));
                    for (int cb = 0; cb < col_blocks; ++cb) {
                        if (edge) tma_load_2d(dst + cb * (row_n * 128) + r0 * 128, map, v_edge, col_lo + cb * 64, row);
                        else tma_load_2d_pair(dst + cb * (row_n * 128) + r0 * 128, map, bar, col_lo + cb * 64, row);
                    }
                }
                if (edge) {
                    if (!mbar_wait(v_edge, edges & 1)) { ok = false; break; }
                    ++edges;
                    if (key0 + PR_BN > ctx) zero_value_rows<PR_BN>(dst, HD / 128, max(0, ctx - key0), PR_BN, 0, 1);
                    if (key0 < key_lo) zero_value_rows<PR_BN>(dst, HD / 128, 0, min(PR_BN, key_lo - key0), 0, 1);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    mbar_arrive_cluster_release(bar);
                }
            }
            for (int k = 0; k < PR_STAGES && ok; ++k, ++n) {          // nothing in flight at the exit
                const int s = n % PR_STAGES, ph = (n / PR_STAGES) & 1;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) ok = false;
            }
            if (!ok) atomicExch(status, GAVE_UP_TC_LOAD);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the first CTA's, for both ----------------
        if (lane == 0 && rank == 0) {
            bool ok = mbar_wait(q_full, 0);
            tc_fence_after();
            auto issue_scores = [&](int n) -> bool {       // S(n) = Q K(n)^T into score buffer n % 2
                const int s = n % PR_STAGES, ph = (n / PR_STAGES) & 1;
                if (!mbar_wait(k_full + 8 * s, ph)) return false;
                tc_fence_after();
                const uint32_t d = tmem_base + TC_S_COL + (n & 1) * PR_BN, kb = k_s + s * PR_K_BYTES;
#pragma unroll
                for (int kt = 0; kt < HD / 16; ++kt)
                    tc_mma_pair(d, smem_desc(q_s + (kt >> 2) * (TC_BM * 128) + (kt & 3) * 32),
                                smem_desc(kb + (kt >> 2) * (64 * 128) + (kt & 3) * 32), IDESC_PR_S, kt > 0 ? 1u : 0u);
                tc_commit_pair(k_empty + 8 * s, 3);
                tc_commit_pair(s_full + 8 * (n & 1), 3);
                return true;
            };
            ok = ok && issue_scores(0);
            for (int n = 0; n < T && ok; ++n) {
                if (n + 1 < T && !issue_scores(n + 1)) { ok = false; break; }
                const int s = n % PR_STAGES, ph = (n / PR_STAGES) & 1;
                if (!mbar_wait(v_full + 8 * s, ph) || !mbar_wait(p_full, n & 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t vb = v_s + s * PR_V_BYTES, pa = tmem_base + TC_S_COL + (n & 1) * PR_BN;
#pragma unroll
                for (int kk = 0; kk < PR_BN / 16; ++kk)
                    tc_mma_ts_pair(tmem_base, pa + kk * 8, smem_desc_mn(vb + kk * (16 * 128), PR_BN * 128), IDESC_PR_PV,
                                   (n > 0 || kk > 0) ? 1u : 0u);
                tc_commit_pair(v_empty + 8 * s, 3);
                tc_commit_pair(pv_done, 3);
            }
            if (!ok) atomicExch(status, GAVE_UP_TC_MMA);
        }
    } else {
        // ---------------- softmax: one thread per row of this CTA ----------------
        const int quarter = warp & 3, row = quarter * 32 + lane, m_row = row0 + row;
        const int epi_tid = threadIdx.x - 64;
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        // this CTA's query rows, in the layout the tensor core reads (the same swizzle as a box copy)
        for (int idx = epi_tid; idx < TC_BM * CPR; idx += 128) {
            const int rr = idx / CPR, chunk = idx % CPR, m = row0 + rr;
            const bool valid = m < rows;
            const bf16* src = valid ? q + (size_t)(q_start + m / rep) * q_stride + (size_t)(g * rep + m % rep) * HD + chunk * 8 : q;
            cp_async16(q_s + swz<TC_BM>(rr, chunk), src, valid);
        }
        cp_commit();
        cp_wait<0>();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lead_q_full);

        const int pos_row = m_row < rows ? pos0 + m_row / rep : -1;            // a row past the end sees no key
        const int first_row = window > 0 ? max(0, pos_row - window + 1) : 0;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int n = 0; n < T; ++n) {
            const int b = n & 1, ph = (n >> 1) & 1, key0 = (t0 + n) * PR_BN;
            if (!mbar_wait(s_full + 8 * b, ph)) { ok = false; break; }
            tc_fence_after();
            uint32_t sv[4][32];
#pragma unroll
            for (int h = 0; h < 4; ++h) tc_ld32(t_lane + TC_S_COL + b * PR_BN + 32 * h, sv[h]);
            tc_wait_ld();
            const bool inner = __all_sync(0xffffffffu, key0 + PR_BN - 1 <= pos_row && key0 >= first_row);
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (inner) {
#pragma unroll
                for (int c = 0; c < PR_BN; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sv[c >> 5][c & 31]));
            } else {
#pragma unroll
                for (int c = 0; c < PR_BN; ++c) {
                    const int key = key0 + c;
                    const float v = (key <= pos_row && key >= first_row) ? __uint_as_float(sv[c >> 5][c & 31]) : -INFINITY;
                    sv[c >> 5][c & 31] = __float_as_uint(v);
                    mx4[c & 3] = fmaxf(mx4[c & 3], v);
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float m_tile = fmaxf(m_run, mx * scale2);
            const float m_new = m_tile > m_run + TC_MAX_SLACK ? m_tile : m_run;      // lazily, as in the kernel above
            const float mbase = m_new == -INFINITY ? 0.f : m_new;
            const float corr = fast_exp2(m_run - mbase);
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t packed[2][32];
#pragma unroll
            for (int c = 0; c < PR_BN; c += 2) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(sv[c >> 5][c & 31]), scale2, -mbase));
                const float p1 = fast_exp2(fmaf(__uint_as_float(sv[(c + 1) >> 5][(c + 1) & 31]), scale2, -mbase));
                sum4[(c >> 1) & 3] += p0 + p1;
                packed[c >> 6][(c >> 1) & 31] = pack_bf16(p0, p1);
            }
            l_run = l_run * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            const bool changed = m_new > m_run;
            m_run = m_new;
            // P over the scores this thread has just read: keys (2j, 2j + 1) in column j of the buffer
            tc_st32(t_lane + TC_S_COL + b * PR_BN, packed[0]);
            tc_st32(t_lane + TC_S_COL + b * PR_BN + 32, packed[1]);
            if (n > 0) {
                if (!mbar_wait(pv_done, (n - 1) & 1)) { ok = false; break; }     // O of the tile before is complete
                tc_fence_after();
                if (__any_sync(0xffffffffu, changed)) {
#pragma unroll 1
                    for (int c0 = 0; c0 < HD; c0 += 32) {
                        uint32_t ov[32];
                        tc_ld32(t_lane + c0, ov);
                        tc_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * corr);
                        tc_st32(t_lane + c0, ov);
                    }
                }
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_p_full);
        }
        if (ok && !mbar_wait(pv_done, (T - 1) & 1)) ok = false;
        ok = __all_sync(0xffffffffu, ok);        // the tensor-memory loads below are collective: all lanes or none
        if (ok) {
            tc_fence_after();
            const float inv = 1.0f / l_run;
            bf16* dst = m_row < rows ? out + (size_t)(q_start + m_row / rep) * out_stride + (size_t)(g * rep + m_row % rep) * HD : nullptr;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t ov[32];
                tc_ld32(t_lane + c0, ov);
                tc_wait_ld();
                if (dst) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 o;
                        o.x = pack_bf16(__uint_as_float(ov[c]) * inv, __uint_as_float(ov[c + 1]) * inv);
                        o.y = pack_bf16(__uint_as_float(ov[c + 2]) * inv, __uint_as_float(ov[c + 3]) * inv);
                        o.z = pack_bf16(__uint_as_float(ov[c + 4]) * inv, __uint_as_float(ov[c + 5]) * inv);
                        o.w = pack_bf16(__uint_as_float(ov[c + 6]) * inv, __uint_as_float(ov[c + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + c) = o;
                    }
                }
            }
        } else if (lane == 0) {
            atomicExch(status, GAVE_UP_TC_SOFTMAX);
        }
    }
    tc_fence_before();
    cluster_sync();                       // nothing of either CTA is still in use by the other
    if (warp == 1) {
        tc_fence_after();
        tc_dealloc_pair(tmem_base, 512);
    }
}
#endif
#endif
