// Sampling of one token per row of logits: greedy, or temperature with top-k, top-p,
// min-p and a repetition penalty, as the reference samples
// (src/wllm/engine/sampling.py:101-143), without a sort.
//
// What is computed, in order:
//   1. repetition penalty, in place, on the row's distinct generated ids:
//      x > 0 ? x / penalty : x * penalty;
//   2. arg-max (lowest id among equals) and log-sum-exp of the penalised row;
//      temperature 0: that arg-max is the token, its log-probability is taken at
//      temperature 1;
//   3. otherwise s = x / max(temperature, 1e-5); the three filters are all judged on
//      softmax(s) of the whole row and each keeps the values at or above a threshold:
//         top-k  the k-th largest value;
//         top-p  the smallest value v with  sum{p_j : s_j >= v} <= top_p;
//         min-p  p_i >= min_p * p_max;
//      the largest value always stays.  Thresholds live on the order-preserving bit
//      pattern of the floats, so equal values are kept or dropped together;
//   4. the token is the first id, in vocabulary order, whose running sum of kept
//      exp(s - max) exceeds u * (their total), with u in [0, 1) hashed from
//      (seed, counter): the draw depends on the request's seed and the place in its
//      output only, not on the batch;
//   5. log-probability of the token under log_softmax(s) before truncation.
//
// How: a row is cut into chunks and every pass runs as a grid of (chunks, rows) blocks,
// so that a row of 256,000 logits is read by up to 64 blocks at a time out of L2.
//   stats     penalty; per chunk: maximum, arg-max, sum of exp.  The last block of a row to
//             finish combines the chunks (greedy rows are done here).
//   select 0..2   the thresholds of top-k and top-p by radix selection on the key: 11, 11 and
//             10 bits a pass.  Each pass builds, per row, a histogram over the next digit of the
//             keys that share the digits found so far (counts for top-k, masses for top-p); the
//             row's last block walks it from the top and fixes the digit.  Pass 0 also finds
//             the lowest key that min-p keeps.
//   draw      per chunk: the kept mass; the row's last block places u * total among the chunks
//             and walks the one chunk that holds it.
// Masses are exp(s - max) in 40-bit fixed point, added as 64-bit integers: sums do not depend
// on their order, so neither the thresholds nor the token depend on how a row was cut or on
// which block came last.  Blocks never wait for one another: "last" is whoever draws the
// final ticket of a per-row counter after publishing its part.
#include "common.cuh"

typedef unsigned long long u64;

constexpr int ST = 256;               // threads a block
constexpr int WARPS = ST / 32;
constexpr int MAX_CHUNKS = 64;
constexpr int BINS = 2048;
constexpr int LEVELS = 3;
constexpr int KEEP = 8;               // vectors of four that a thread of the stats pass keeps in registers
constexpr float MASS_ONE = 1099511627776.0f;      // 2^40

// Per-row scratch: this state, then the chunks' statistics, the kept masses of their segments and the histograms.
struct RowState {
    unsigned done[5];        // tickets: stats, select 0..2, draw; each returns to 0 when its pass is over
    unsigned searching;      // bit 0: top-k still has digits to find; bit 1: top-p; bit 2: min-p is asked for
    unsigned greedy;
    int best_i;
    float xmax, log_z, inv_t;
    unsigned min_p_key, prefix_k, prefix_p, rem_k, thr_k, thr_p;
    u64 rem_p;
};
constexpr size_t STATE_BYTES = 128;
constexpr size_t STATS_BYTES = MAX_CHUNKS * 3 * sizeof(float);
constexpr size_t SEGMENT_BYTES = MAX_CHUNKS * WARPS * sizeof(u64);
constexpr size_t COUNT_BYTES = (size_t)LEVELS * BINS * sizeof(unsigned);
constexpr size_t MASS_BYTES = (size_t)LEVELS * BINS * sizeof(u64);
constexpr size_t ROW_BYTES = STATE_BYTES + STATS_BYTES + SEGMENT_BYTES + COUNT_BYTES + MASS_BYTES;
static_assert(sizeof(RowState) <= STATE_BYTES && ROW_BYTES % 16 == 0, "row scratch layout");

struct RowScratch {
    RowState* state;
    float* stats;
    u64* segment_mass;   // [chunks][WARPS]
    unsigned* counts;    // [LEVELS][BINS]
    u64* masses;         // [LEVELS][BINS]
};
__device__ __forceinline__ RowScratch row_scratch(unsigned char* scratch, int row) {
    unsigned char* p = scratch + (size_t)row * ROW_BYTES;
    RowScratch r;
    r.state = reinterpret_cast<RowState*>(p);
    r.stats = reinterpret_cast<float*>(p + STATE_BYTES);
    r.segment_mass = reinterpret_cast<u64*>(p + STATE_BYTES + STATS_BYTES);
    r.counts = reinterpret_cast<unsigned*>(p + STATE_BYTES + STATS_BYTES + SEGMENT_BYTES);
    r.masses = reinterpret_cast<u64*>(p + STATE_BYTES + STATS_BYTES + SEGMENT_BYTES + COUNT_BYTES);
    return r;
}

// Rows are cut at multiples of four, so that a chunk of an aligned row is read four values at a time.
__device__ __forceinline__ int chunk_length(int V, int chunks) { return (((V + chunks - 1) / chunks) + 3) & ~3; }
__device__ __forceinline__ bool row_is_aligned(const float* x) { return ((uintptr_t)x & 15) == 0; }

// f(i, x[i]) for every i of [lo, hi), the block's threads side by side; lo is a multiple of four.
template <typename F>
__device__ __forceinline__ void for_each_of_chunk(const float* __restrict__ x, int lo, int hi, bool aligned, F f) {
    if (aligned) {
#pragma unroll 2
        for (int i = lo + threadIdx.x * 4; i < hi; i += ST * 4) {
            if (i + 4 <= hi) {
                const float4 t = *reinterpret_cast<const float4*>(x + i);
                f(i, t.x); f(i + 1, t.y); f(i + 2, t.z); f(i + 3, t.w);
            } else {
                for (int j = i; j < hi; ++j) f(j, x[j]);
            }
        }
    } else {
#pragma unroll 4
        for (int i = lo + threadIdx.x; i < hi; i += ST) f(i, x[i]);
    }
}

__device__ __forceinline__ unsigned key_of(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
// exp(s - s_max) of s = x / T, as 2^((x - x_max) * log2(e) / T) by the hardware's exponential (relative error
// 2^-22: every pass uses this one function, so they agree with one another exactly), and the same in 40-bit
// fixed point
__device__ __forceinline__ float weight_of(float x, float xmax, float inv_t) {
    const float c = inv_t * 1.4426950408889634f;
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(fmaf(x, c, -(xmax * c))));
    return y;
}
__device__ __forceinline__ u64 mass_of(float x, float xmax, float inv_t) { return __float2ull_rd(weight_of(x, xmax, inv_t) * MASS_ONE); }

// The float whose key is `key`, and bounds lo <= x <= hi that hold for every x whose key lies in
// [first, last] (they may hold for a few more: -0 and +0 compare equal but have different keys).
__device__ __forceinline__ float float_of_key(unsigned key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}
__device__ __forceinline__ void bounds_of_keys(unsigned first, unsigned last, float& lo, float& hi) {
    lo = float_of_key(first);
    hi = float_of_key(last);
    if (lo != lo) lo = -INFINITY;     // the ends of the key range are not-a-number patterns
    if (hi != hi) hi = INFINITY;
}

__device__ __forceinline__ unsigned uniform_bits(unsigned long long seed, unsigned long long counter) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (counter + 1ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (unsigned)(z >> 40);     // u = bits / 2^24
}

__device__ __forceinline__ u64 warp_inclusive_scan(u64 v) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 up = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += up;
    }
    return v;
}

// Sum of v over the block and, for each thread, the sum over the threads before it.
__device__ __forceinline__ u64 block_scan(u64 v, u64* warp_totals, u64& total) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const u64 inc = warp_inclusive_scan(v);
    __syncthreads();
    if (lane == 31) warp_totals[warp] = inc;
    __syncthreads();
    u64 before = inc - v;
    total = 0;
    for (int w = 0; w < WARPS; ++w) {
        const u64 t = warp_totals[w];
        if (w < warp) before += t;
        total += t;
    }
    return before;
}

// True in every thread of the block that drew the last of `tickets` tickets of `counter`.  What the other
// blocks wrote before they drew theirs is visible to that block; the counter is back at 0 then.
__device__ __forceinline__ bool last_block(unsigned* counter, unsigned tickets, int* flag) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool last = atomicAdd(counter, 1u) == tickets - 1;
        if (last) { *counter = 0u; __threadfence(); }
        *flag = last;
    }
    __syncthreads();
    return *flag != 0;
}

__device__ __forceinline__ void take_better(float& best, int& best_i, float v, int i) {
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
}
// arg-max over the block, lowest id among equals; every thread gets the result
__device__ __forceinline__ void block_argmax(float& best, int& best_i, float* fs, int* is) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        take_better(best, best_i, ov, oi);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { fs[threadIdx.x >> 5] = best; is[threadIdx.x >> 5] = best_i; }
    __syncthreads();
    best = fs[0]; best_i = is[0];
    for (int w = 1; w < WARPS; ++w) take_better(best, best_i, fs[w], is[w]);
}

// ------------------------------------------------------------------------------------------------
// stats
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(ST)
sample_stats_kernel(float* __restrict__ logits, int row_stride, int V, unsigned char* __restrict__ scratch,
                    const float* __restrict__ temperature, const int* __restrict__ top_k, const float* __restrict__ top_p,
                    const float* __restrict__ min_p, const float* __restrict__ penalty, const int* __restrict__ gen_offsets,
                    const int* __restrict__ gen_ids, int* __restrict__ out_token, float* __restrict__ out_logprob) {
    __shared__ float fs[32];
    __shared__ int is[32];
    __shared__ int flag;
    pdl_begin();
    const int chunk = blockIdx.x, chunks = gridDim.x, row = blockIdx.y, tid = threadIdx.x;
    const int per = chunk_length(V, chunks);
    const int lo = min(V, chunk * per), hi = min(V, lo + per);
    float* x = logits + (size_t)row * row_stride;
    const bool aligned = row_is_aligned(x);
    const RowScratch rs = row_scratch(scratch, row);

    // without options every row is greedy and unpenalised
    const float temp = temperature ? temperature[row] : 0.0f;
    const bool greedy = temp == 0.0f;
    const float inv_t = greedy ? 1.0f : 1.0f / fmaxf(temp, 1e-5f);
    const int k = greedy ? 0 : top_k[row];
    const bool want_k = !greedy && k > 0 && k < V, want_p = !greedy && top_p[row] < 1.0f;
    if (want_k || want_p) {      // this block's share of the row's histograms
        const int n = LEVELS * BINS, share = (n + chunks - 1) / chunks;
        for (int i = chunk * share + tid; i < min(n, (chunk + 1) * share); i += ST) { rs.counts[i] = 0u; rs.masses[i] = 0ull; }
    }

    const float pen = penalty ? penalty[row] : 1.0f;
    if (pen != 1.0f) {
        for (int i = gen_offsets[row] + tid; i < gen_offsets[row + 1]; i += ST) {
            const int id = gen_ids[i];
            if (id >= lo && id < hi) {
                const float v = x[id];
                x[id] = v > 0.f ? v / pen : v * pen;
            }
        }
        __syncthreads();
    }

    float best = -INFINITY, z = 0.f;
    int best_i = V;
    if (aligned && hi - lo <= ST * 4 * KEEP) {
        // the chunk stays in registers between the maximum and the sum
        float4 v[KEEP];
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = lo + (j * ST + tid) * 4;
            v[j] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            if (i + 4 <= hi) v[j] = *reinterpret_cast<const float4*>(x + i);
            else if (i < hi) { v[j].x = x[i]; if (i + 1 < hi) v[j].y = x[i + 1]; if (i + 2 < hi) v[j].z = x[i + 2]; }
        }
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = lo + (j * ST + tid) * 4;
            if (v[j].x > best) { best = v[j].x; best_i = i; }
            if (v[j].y > best) { best = v[j].y; best_i = i + 1; }
            if (v[j].z > best) { best = v[j].z; best_i = i + 2; }
            if (v[j].w > best) { best = v[j].w; best_i = i + 3; }
        }
        block_argmax(best, best_i, fs, is);
        __syncthreads();
#pragma unroll
        for (int j = 0; j < KEEP; ++j)      // what lies past the chunk's end is -inf and adds 0
            z += (weight_of(v[j].x, best, inv_t) + weight_of(v[j].y, best, inv_t)) + (weight_of(v[j].z, best, inv_t) + weight_of(v[j].w, best, inv_t));
        if (best == -INFINITY) z = 0.f;     // an empty chunk
    } else {
        for_each_of_chunk(x, lo, hi, aligned, [&](int i, float v) { if (v > best) { best = v; best_i = i; } });
        block_argmax(best, best_i, fs, is);
        __syncthreads();
        const float m = best;
        for_each_of_chunk(x, lo, hi, aligned, [&](int, float v) { z += weight_of(v, m, inv_t); });
    }
    z = block_sum(z, fs);
    if (tid == 0) { rs.stats[chunk * 3] = best; rs.stats[chunk * 3 + 1] = __int_as_float(best_i); rs.stats[chunk * 3 + 2] = z; }

    if (!last_block(&rs.state->done[0], chunks, &flag)) return;
    if (tid < 32) {        // the chunks combined in chunk order, two to a lane
        float m[2], zc[2];
        int bi[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c = tid * 2 + j;
            m[j] = c < chunks ? __ldcg(rs.stats + c * 3) : -INFINITY;
            bi[j] = c < chunks ? __float_as_int(__ldcg(rs.stats + c * 3 + 1)) : V;
            zc[j] = c < chunks ? __ldcg(rs.stats + c * 3 + 2) : 0.f;
        }
        float b = m[0];
        int b_i = bi[0];
        take_better(b, b_i, m[1], bi[1]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, b, o);
            const int oi = __shfl_xor_sync(0xffffffffu, b_i, o);
            take_better(b, b_i, ov, oi);
        }
        float total = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j) total += zc[j] == 0.f ? 0.f : zc[j] * weight_of(m[j], b, inv_t);   // an empty chunk: max -inf, sum 0
        total = warp_sum(total);
        if (tid == 0) {
            RowState* s = rs.state;
            const float log_z = logf(total);
            s->greedy = greedy;
            s->best_i = b_i;
            s->xmax = b; s->log_z = log_z; s->inv_t = inv_t;
            const bool want_min = !greedy && min_p[row] > 0.0f;
            s->searching = (want_k ? 1u : 0u) | (want_p ? 2u : 0u) | (want_min ? 4u : 0u);
            s->min_p_key = want_min ? 0xffffffffu : 0u;
            s->prefix_k = s->prefix_p = 0u;
            s->rem_k = want_k ? (unsigned)k : 0u;
            s->rem_p = 0ull;
            s->thr_k = s->thr_p = 0u;
            if (greedy) { out_token[row] = b_i; out_logprob[row] = -log_z; }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// select: one digit of the top-k and top-p thresholds
// ------------------------------------------------------------------------------------------------
template <int LEVEL> __device__ __forceinline__ unsigned digit_of(unsigned key) {
    return LEVEL == 0 ? key >> 21 : (LEVEL == 1 ? (key >> 10) & 2047u : key & 1023u);
}
template <int LEVEL> __device__ __forceinline__ unsigned above_of(unsigned key) {   // the digits before this level's
    return LEVEL == 0 ? 0u : (LEVEL == 1 ? key >> 21 : key >> 10);
}
template <int LEVEL> __device__ __forceinline__ unsigned place(unsigned digit) {
    return LEVEL == 0 ? digit << 21 : (LEVEL == 1 ? digit << 10 : digit);
}

template <int LEVEL>
__global__ void __launch_bounds__(ST)
sample_select_kernel(const float* __restrict__ logits, int row_stride, int V, unsigned char* __restrict__ scratch,
                     const float* __restrict__ top_p, const float* __restrict__ min_p) {
    // Pass 0 sees every value, most of them in a few bins: it counts in shared memory first.  A bin's mass is
    // held there as two 32-bit halves, which shared memory adds in one instruction.  The later passes see
    // the few values that share the digits found so far and add them to the row's histogram directly.
    constexpr int LOCAL = LEVEL == 0 ? BINS : 4;
    __shared__ __align__(16) unsigned hc[LOCAL], hm_lo[LOCAL], hm_hi[LOCAL];
    __shared__ u64 warp_totals[WARPS];
    __shared__ unsigned us[32];
    __shared__ int flag;
    pdl_begin();
    const int chunk = blockIdx.x, chunks = gridDim.x, row = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    const RowScratch rs = row_scratch(scratch, row);
    RowState* s = rs.state;
    const unsigned searching = s->searching;
    const bool do_k = searching & 1u, do_p = searching & 2u, do_min = LEVEL == 0 && (searching & 4u);
    if (!do_k && !do_p && !do_min) return;
    const int per = chunk_length(V, chunks);
    const int lo = min(V, chunk * per), hi = min(V, lo + per);
    const float* x = logits + (size_t)row * row_stride;
    const float inv_t = s->inv_t, xmax = s->xmax;
    const unsigned above_k = above_of<LEVEL>(s->prefix_k), above_p = above_of<LEVEL>(s->prefix_p);
    const float p_min = min_p[row];
    unsigned* gc = rs.counts + LEVEL * BINS;
    u64* gm = rs.masses + LEVEL * BINS;
    unsigned lowest = 0xffffffffu;

    if (LEVEL == 0) {
        for (int b = tid * 4; b < BINS; b += ST * 4) {
            *reinterpret_cast<uint4*>(hc + b) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(hm_lo + b) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(hm_hi + b) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncthreads();
        for_each_of_chunk(x, lo, hi, row_is_aligned(x), [&](int, float v) {
            const unsigned key = key_of(v);
            const unsigned d = digit_of<LEVEL>(key);
            if (do_k) atomicAdd(&hc[d], 1u);
            if (do_p || do_min) {
                const float w = weight_of(v, xmax, inv_t);
                if (do_p) {
                    const u64 m = __float2ull_rd(w * MASS_ONE);
                    const unsigned ml = (unsigned)m, mh = (unsigned)(m >> 32);
                    if (ml) {
                        const unsigned old = atomicAdd(&hm_lo[d], ml);
                        if (old + ml < old) atomicAdd(&hm_hi[d], 1u);      // this addition wrapped the lower half
                    }
                    if (mh) atomicAdd(&hm_hi[d], mh);
                }
                // p_i < min_p * p_max is dropped  <=>  exp(s_i - s_max) < min_p; the keys are monotone in s
                if (do_min && !(w < p_min)) lowest = min(lowest, key);
            }
        });
        __syncthreads();
        for (int b = tid * 4; b < BINS; b += ST * 4) {
            const uint4 c4 = *reinterpret_cast<const uint4*>(hc + b);
            const uint4 l4 = *reinterpret_cast<const uint4*>(hm_lo + b), h4 = *reinterpret_cast<const uint4*>(hm_hi + b);
            const unsigned cs[4] = {c4.x, c4.y, c4.z, c4.w}, ls[4] = {l4.x, l4.y, l4.z, l4.w}, hs[4] = {h4.x, h4.y, h4.z, h4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (cs[j]) atomicAdd(gc + b + j, cs[j]);
                const u64 m = ((u64)hs[j] << 32) | ls[j];
                if (m) atomicAdd(gm + b + j, m);
            }
        }
    } else {
        // Values outside the bins found so far fail two comparisons of floats and cost nothing more.
        constexpr unsigned width = LEVEL == 1 ? (1u << 21) : (1u << 10);
        float k_lo, k_hi, p_lo, p_hi;
        bounds_of_keys(place<LEVEL - 1>(above_k) , place<LEVEL - 1>(above_k) + (width - 1u), k_lo, k_hi);
        bounds_of_keys(place<LEVEL - 1>(above_p), place<LEVEL - 1>(above_p) + (width - 1u), p_lo, p_hi);
        for_each_of_chunk(x, lo, hi, row_is_aligned(x), [&](int, float v) {
            const bool near_k = do_k && v >= k_lo && v <= k_hi, near_p = do_p && v >= p_lo && v <= p_hi;
            if (near_k || near_p) {
                const unsigned key = key_of(v);
                const unsigned d = digit_of<LEVEL>(key), a = above_of<LEVEL>(key);
                if (near_k && a == above_k) {       // one addition for the lanes of a warp that meet in a bin
                    const unsigned peers = __match_any_sync(__activemask(), d);
                    if (lane == __ffs(peers) - 1) atomicAdd(gc + d, (unsigned)__popc(peers));
                }
                if (near_p && a == above_p) {
                    const u64 m = mass_of(v, xmax, inv_t);
                    const unsigned peers = __match_any_sync(__activemask(), d);
                    u64 sum = 0;
                    for (unsigned rest = peers; rest; rest &= rest - 1) sum += __shfl_sync(peers, m, __ffs(rest) - 1);
                    if (lane == __ffs(peers) - 1 && sum) atomicAdd(gm + d, sum);
                }
            }
        });
    }
    if (do_min) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lowest = min(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
        if ((tid & 31) == 0) us[tid >> 5] = lowest;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < WARPS; ++w) lowest = min(lowest, us[w]);
            atomicMin(&s->min_p_key, lowest);
        }
    }
    if (!last_block(&s->done[1 + LEVEL], chunks, &flag)) return;
    if (!do_k && !do_p) {
        if (tid == 0) s->searching = 0u;
        return;
    }

    // The row's histogram, walked from the top: thread t holds bins BINS-1-8t down to BINS-8-8t.
    constexpr int PER = BINS / ST;
    unsigned c[PER];
    u64 m[PER];
    u64 c_sum = 0, m_sum = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int b = BINS - 1 - (tid * PER + j);
        c[j] = do_k ? __ldcg(gc + b) : 0u;
        m[j] = do_p ? __ldcg(gm + b) : 0ull;
        c_sum += c[j]; m_sum += m[j];
    }
    u64 c_total, m_total;
    const u64 c_before = block_scan(c_sum, warp_totals, c_total);
    const u64 m_before = block_scan(m_sum, warp_totals, m_total);
    // kept <=> the mass at or above it <= top_p * total: integers on both sides
    u64 budget = s->rem_p;
    if (LEVEL == 0 && do_p) budget = __double2ull_rd((double)top_p[row] * (double)m_total);
    constexpr bool final_level = LEVEL == LEVELS - 1;
    if (do_k) {
        // the digit of the k-th largest key: the first bin from the top at which the count reaches what is left of k
        const u64 want = s->rem_k;
        if (c_before < want && want <= c_before + c_sum) {
            u64 run = c_before;
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                if (run < want && want <= run + c[j]) {
                    const unsigned prefix = s->prefix_k | place<LEVEL>((unsigned)(BINS - 1 - (tid * PER + j)));
                    s->prefix_k = prefix;
                    s->rem_k = (unsigned)(want - run);
                    if (final_level) s->thr_k = prefix;
                }
                run += c[j];
            }
        }
    }
    if (do_p) {
        // the digit of the largest key whose mass at or above it exceeds the budget; the threshold is the next key up
        if (m_total <= budget) {
            if (tid == 0) { s->thr_p = 0u; s->searching = searching & ~2u; }    // everything fits: top-p drops nothing
        } else if (m_before <= budget && budget < m_before + m_sum) {
            u64 run = m_before;
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                if (run <= budget && budget < run + m[j]) {
                    const unsigned prefix = s->prefix_p | place<LEVEL>((unsigned)(BINS - 1 - (tid * PER + j)));
                    s->prefix_p = prefix;
                    s->rem_p = budget - run;
                    if (final_level) s->thr_p = prefix == 0xffffffffu ? prefix : prefix + 1u;
                }
                run += m[j];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// draw
// ------------------------------------------------------------------------------------------------
// A chunk is cut once more into one contiguous segment a warp; a warp reads its segment 32 neighbouring
// values at a time.
__device__ __forceinline__ int segment_length(int per) { return (per + WARPS - 1) / WARPS; }

__global__ void __launch_bounds__(ST)
sample_draw_kernel(const float* __restrict__ logits, int row_stride, int V, unsigned char* __restrict__ scratch,
                   const int* __restrict__ seed_lo, const int* __restrict__ seed_hi, const int* __restrict__ counter,
                   int* __restrict__ out_token, float* __restrict__ out_logprob) {
    __shared__ u64 warp_totals[WARPS];
    constexpr int STAGED = 2048;
    __shared__ float segment[STAGED];
    __shared__ u64 home_before;
    __shared__ int home;
    __shared__ int flag;
    pdl_begin();
    const int chunk = blockIdx.x, chunks = gridDim.x, row = blockIdx.y, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const RowScratch rs = row_scratch(scratch, row);
    RowState* s = rs.state;
    if (s->greedy) return;
    const int per = chunk_length(V, chunks), seg = segment_length(per);
    const float* x = logits + (size_t)row * row_stride;
    const float inv_t = s->inv_t, xmax = s->xmax;
    // the largest value always stays
    const unsigned threshold = min(max(max(s->thr_k, s->thr_p), s->min_p_key), key_of(xmax));
    {
        const int c_hi = min(V, (chunk + 1) * per);
        const int lo = min(c_hi, chunk * per + warp * seg), hi = min(c_hi, lo + seg);
        u64 local = 0;
#pragma unroll 4
        for (int i = lo + lane; i < hi; i += 32) {
            const float v = x[i];
            if (key_of(v) >= threshold) local += mass_of(v, xmax, inv_t);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
        if (lane == 0) rs.segment_mass[chunk * WARPS + warp] = local;
    }
    if (!last_block(&s->done[4], chunks, &flag)) return;

    // Where u * total falls among the segments (chunks * WARPS of them, at most two a thread), then inside
    // that segment.
    const int segments = chunks * WARPS;
    u64 mine[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) mine[j] = tid * 2 + j < segments ? __ldcg(rs.segment_mass + tid * 2 + j) : 0ull;
    u64 total;
    const u64 before = block_scan(mine[0] + mine[1], warp_totals, total);
    if (total == 0ull) {       // nothing but not-a-numbers in the row: the arg-max stands in
        if (tid == 0) { out_token[row] = min(s->best_i, V - 1); out_logprob[row] = -s->log_z; }
        return;
    }
    const u64 seed = ((u64)(unsigned)seed_hi[row] << 32) | (unsigned)seed_lo[row];
    const u64 bits = uniform_bits(seed, (u64)(unsigned)counter[row]);
    // floor(total * bits / 2^24), below total since bits < 2^24
    const u64 target = (__umul64hi(total, bits) << 40) | ((total * bits) >> 24);
    if (before <= target && target < before + mine[0]) { home = tid * 2; home_before = before; }
    else if (before + mine[0] <= target && target < before + mine[0] + mine[1]) { home = tid * 2 + 1; home_before = before + mine[0]; }
    __syncthreads();
    const int h_chunk = home / WARPS, h_warp = home % WARPS;
    const int c_hi = min(V, (h_chunk + 1) * per);
    const int lo = min(c_hi, h_chunk * per + h_warp * seg), hi = min(c_hi, lo + seg);
    // The segment comes into shared memory with all its loads in flight at once; one warp then walks it.
    const bool staged = hi - lo <= STAGED;
    if (staged) {
        for (int i = tid; i < hi - lo; i += ST) segment[i] = x[lo + i];
        __syncthreads();
    }
    if (warp != 0) return;
    u64 run = home_before;
    for (int base = lo; base < hi; base += 32) {
        const int i = base + lane;
        u64 m = 0;
        float v = 0.f;
        if (i < hi) {
            v = staged ? segment[i - lo] : x[i];
            if (key_of(v) >= threshold) m = mass_of(v, xmax, inv_t);
        }
        const u64 inc = run + warp_inclusive_scan(m);
        const unsigned hit = __ballot_sync(0xffffffffu, inc > target);
        if (hit) {
            if (lane == __ffs(hit) - 1) { out_token[row] = i; out_logprob[row] = (v - xmax) * inv_t - s->log_z; }
            return;
        }
        run = __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) { out_token[row] = min(s->best_i, V - 1); out_logprob[row] = -s->log_z; }   // not reached: the sums are exact
}

// 64 blocks a row for few rows, 32 for more: fewer (16, 8) measured slower at every number of rows, the
// last block's share growing with the chunk.
static int chunks_for(int rows) { return rows <= 8 ? 64 : 32; }

// Greedy tokens and their log-probabilities (temperature 1) for `rows` rows without a penalty: the stats pass
// alone, with no options to read.  `scratch` as for wllm_sample.
WLLM_API int wllm_sample_greedy(float* logits, int row_stride, int rows, int V, void* scratch, int* out_token,
                                float* out_logprob, cudaStream_t stream) {
    if (rows <= 0) return WLLM_OK;
    if (V <= 0 || row_stride < V || rows > 65535) return WLLM_BAD_SIZE;
    if (!scratch || ((uintptr_t)scratch & 15)) return WLLM_BAD_ALIGN;
    const float* none_f = nullptr;
    const int* none_i = nullptr;
    return wllm_launch(sample_stats_kernel, dim3(chunks_for(rows), rows), ST, 0, stream, logits, row_stride, V,
                       (unsigned char*)scratch, none_f, none_i, none_f, none_f, none_f, none_i, none_i, out_token, out_logprob);
}

// Bytes of scratch that wllm_sample needs for each row.  The scratch must be zero before its first use;
// every call leaves it ready for the next.
WLLM_API int wllm_sample_scratch_row_bytes() { return (int)ROW_BYTES; }

// `filters`: bit 0 set when some row asks for top-k, top-p or min-p (the first selection pass runs), bit 1
// when some row asks for top-k or top-p (the two further passes run).  Rows decide for themselves from their
// own options; the bits only leave out launches that would find nothing to do.
WLLM_API int wllm_sample(float* logits, int row_stride, int rows, int V, const float* temperature, const int* top_k,
                         const float* top_p, const float* min_p, const float* penalty, const int* seed_lo,
                         const int* seed_hi, const int* counter, const int* gen_offsets, const int* gen_ids,
                         void* scratch, int filters, int* out_token, float* out_logprob, int* launched,
                         cudaStream_t stream) {
    if (launched) *launched = 0;
    if (rows <= 0) return WLLM_OK;
    if (V <= 0 || row_stride < V || rows > 65535) return WLLM_BAD_SIZE;
    if (!scratch || ((uintptr_t)scratch & 15)) return WLLM_BAD_ALIGN;
    const int chunks = chunks_for(rows);
    const dim3 grid(chunks, rows);
    unsigned char* sc = (unsigned char*)scratch;
    int n = 0;
    int st = wllm_launch(sample_stats_kernel, grid, ST, 0, stream, logits, row_stride, V, sc, temperature, top_k, top_p, min_p,
                         penalty, gen_offsets, gen_ids, out_token, out_logprob);
    ++n;
    if (!st && (filters & 1)) { st = wllm_launch(sample_select_kernel<0>, grid, ST, 0, stream, (const float*)logits, row_stride, V, sc, top_p, min_p); ++n; }
    if (!st && (filters & 2)) { st = wllm_launch(sample_select_kernel<1>, grid, ST, 0, stream, (const float*)logits, row_stride, V, sc, top_p, min_p); ++n; }
    if (!st && (filters & 2)) { st = wllm_launch(sample_select_kernel<2>, grid, ST, 0, stream, (const float*)logits, row_stride, V, sc, top_p, min_p); ++n; }
    if (!st) { st = wllm_launch(sample_draw_kernel, grid, ST, 0, stream, (const float*)logits, row_stride, V, sc, seed_lo, seed_hi, counter, out_token, out_logprob); ++n; }
    if (launched) *launched = n;
    return st;
}
