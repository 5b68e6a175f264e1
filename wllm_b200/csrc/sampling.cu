// Sampling of one token per row of logits: greedy, or temperature with top-k, top-p,
// min-p and a repetition penalty, as the reference samples
// (src/wllm/engine/sampling.py:101-143), without a sort.
//
// One block per row.  In order:
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
//      the largest value always stays.  Thresholds are found by bisection on the
//      order-preserving bit pattern of the floats (32 passes over the row, which sits
//      in L2), so equal values are kept or dropped together;
//   4. the token is the first id, in vocabulary order, whose running sum of kept
//      exp(s - max) exceeds u * (their total), with u in [0, 1) hashed from
//      (seed, counter): the draw depends on the request's seed and the place in its
//      output only, not on the batch;
//   5. log-probability of the token under log_softmax(s) before truncation.
#include "common.cuh"

constexpr int THREADS = 1024;

__device__ __forceinline__ unsigned key_of(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float uniform_from(unsigned long long seed, unsigned long long counter) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (counter + 1ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ unsigned block_count(unsigned v, unsigned* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    unsigned total = 0;
    for (int w = 0; w < THREADS / 32; ++w) total += scratch[w];
    return total;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(float* __restrict__ logits, int row_stride, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ penalty, const int* __restrict__ seed_lo, const int* __restrict__ seed_hi,
              const int* __restrict__ counter, const int* __restrict__ gen_offsets, const int* __restrict__ gen_ids,
              int* __restrict__ out_token, float* __restrict__ out_logprob) {
    __shared__ float fscratch[32];
    __shared__ unsigned uscratch[32];
    __shared__ int ibest[32];
    __shared__ float chunk_sums[THREADS];
    __shared__ int chosen;
    pdl_begin();
    const int row = blockIdx.x, tid = threadIdx.x;
    float* x = logits + (size_t)row * row_stride;

    // 1. repetition penalty on distinct ids
    const float pen = penalty[row];
    if (pen != 1.0f) {
        for (int i = gen_offsets[row] + tid; i < gen_offsets[row + 1]; i += THREADS) {
            const int id = gen_ids[i];
            if (id >= 0 && id < V) {
                const float v = x[id];
                x[id] = v > 0.f ? v / pen : v * pen;
            }
        }
        __syncthreads();
    }

    // 2. arg-max, lowest id among equals
    float best = -INFINITY;
    int best_i = V;
    for (int i = tid; i < V; i += THREADS) {
        const float v = x[i];
        if (v > best) { best = v; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((tid & 31) == 0) { fscratch[tid >> 5] = best; ibest[tid >> 5] = best_i; }
    __syncthreads();
    best = fscratch[0]; best_i = ibest[0];
    for (int w = 1; w < THREADS / 32; ++w)
        if (fscratch[w] > best || (fscratch[w] == best && ibest[w] < best_i)) { best = fscratch[w]; best_i = ibest[w]; }
    __syncthreads();

    const float temp = temperature[row];
    const bool greedy = temp == 0.0f;
    const float T = greedy ? 1.0f : fmaxf(temp, 1e-5f);
    const float smax = best / T;

    float z = 0.f;
    for (int i = tid; i < V; i += THREADS) z += expf(x[i] / T - smax);
    z = block_sum(z, fscratch);
    const float log_z = logf(z);

    if (greedy) {
        if (tid == 0) { out_token[row] = best_i; out_logprob[row] = -log_z; }
        return;
    }

    // 3. thresholds on the order-preserving keys of s = x / T
    const unsigned key_max = key_of(smax);
    unsigned threshold = 0u;
    const int k = top_k[row];
    if (k > 0 && k < V) {
        unsigned t = 0u;   // largest t with count(key >= t) >= k, i.e. the k-th largest key
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = t | (1u << bit);
            unsigned c = 0;
            for (int i = tid; i < V; i += THREADS) c += key_of(x[i] / T) >= cand;
            if (block_count(c, uscratch) >= (unsigned)k) t = cand;
        }
        threshold = max(threshold, t);
    }
    const float p_top = top_p[row];
    if (p_top < 1.0f) {
        unsigned t = 0u;   // largest t whose kept mass still exceeds top_p; the answer is t + 1
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = t | (1u << bit);
            float s = 0.f;
            for (int i = tid; i < V; i += THREADS) {
                const float v = x[i] / T;
                if (key_of(v) >= cand) s += expf(v - smax);
            }
            if (block_sum(s, fscratch) / z > p_top) t = cand;
        }
        threshold = max(threshold, t == 0xffffffffu ? t : t + 1u);
    }
    const float p_min = min_p[row];
    if (p_min > 0.0f) {
        // p_i < min_p * p_max is dropped  <=>  exp(s_i - smax) < min_p
        unsigned t = 0u;   // largest t such that some dropped key is >= t ... found directly instead:
        // keys are monotone in s, so the smallest kept key is the smallest key with exp(s - smax) >= min_p
        unsigned lowest = 0xffffffffu;
        for (int i = tid; i < V; i += THREADS) {
            const float v = x[i] / T;
            if (!(expf(v - smax) / z < p_min * (1.0f / z))) lowest = min(lowest, key_of(v));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lowest = min(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
        __syncthreads();
        if ((tid & 31) == 0) uscratch[tid >> 5] = lowest;
        __syncthreads();
        t = 0xffffffffu;
        for (int w = 0; w < THREADS / 32; ++w) t = min(t, uscratch[w]);
        __syncthreads();
        threshold = max(threshold, t);
    }
    threshold = min(threshold, key_max);   // the largest value always stays

    // 4. inverse CDF over the kept values, in vocabulary order: thread t owns a contiguous chunk
    const int chunk = (V + THREADS - 1) / THREADS;
    const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);
    float local = 0.f;
    for (int i = lo; i < hi; ++i) {
        const float v = x[i] / T;
        if (key_of(v) >= threshold) local += expf(v - smax);
    }
    chunk_sums[tid] = local;
    if (tid == 0) chosen = -1;
    __syncthreads();
    if (tid == 0) {   // serial scan of 1024 partial sums: a fixed order, and cheap beside the passes above
        float run = 0.f;
        for (int t2 = 0; t2 < THREADS; ++t2) { const float c = chunk_sums[t2]; chunk_sums[t2] = run; run += c; }
        fscratch[0] = run;
    }
    __syncthreads();
    const float total = fscratch[0];
    const unsigned long long seed = ((unsigned long long)(unsigned)seed_hi[row] << 32) | (unsigned)seed_lo[row];
    const float target = uniform_from(seed, (unsigned long long)(unsigned)counter[row]) * total;
    const float before = chunk_sums[tid];
    if (local > 0.f && target >= before && target < before + local) {
        float run = before;
        int pick = -1, last_kept = -1;
        for (int i = lo; i < hi; ++i) {
            const float v = x[i] / T;
            if (key_of(v) >= threshold) {
                last_kept = i;
                run += expf(v - smax);
                if (run > target) { pick = i; break; }
            }
        }
        chosen = pick >= 0 ? pick : last_kept;
    }
    __syncthreads();
    if (tid == 0) {
        int tok = chosen;
        if (tok < 0) tok = best_i;   // rounding put the target at or past the total: the largest value stands in
        out_token[row] = tok;
        out_logprob[row] = (x[tok] / T - smax) - log_z;
    }
}

// ------------------------------------------------------------------------------------------------
// greedy rows without a penalty: two short kernels instead of one block per row
// ------------------------------------------------------------------------------------------------
// Stage 1, grid (chunks, rows): arg-max (lowest id among equals), maximum and sum of exp(x - max) of one
// chunk of a row.  Stage 2, one warp per row: the chunks' results combined in chunk order.  A row of
// 256,000 logits is read once, by 32 blocks instead of one.
constexpr int GREEDY_CHUNKS = 32;

__global__ void __launch_bounds__(256)
greedy_stats_kernel(const float* __restrict__ logits, int row_stride, int V, float* __restrict__ stats) {
    __shared__ float fs[32];
    __shared__ int is[32];
    pdl_begin();
    const int chunk = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
    const int per = (V + GREEDY_CHUNKS - 1) / GREEDY_CHUNKS;
    const int lo = chunk * per, hi = min(V, lo + per);
    const float* x = logits + (size_t)row * row_stride;
    float best = -INFINITY;
    int best_i = V;
    for (int i = lo + tid; i < hi; i += 256) {
        const float v = x[i];
        if (v > best) { best = v; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((tid & 31) == 0) { fs[tid >> 5] = best; is[tid >> 5] = best_i; }
    __syncthreads();
    best = fs[0]; best_i = is[0];
    for (int w = 1; w < 8; ++w)
        if (fs[w] > best || (fs[w] == best && is[w] < best_i)) { best = fs[w]; best_i = is[w]; }
    __syncthreads();
    float z = 0.f;
    for (int i = lo + tid; i < hi; i += 256) z += expf(x[i] - best);
    z = block_sum(z, fs);
    if (tid == 0) {
        float* out = stats + ((size_t)row * GREEDY_CHUNKS + chunk) * 3;
        out[0] = best; out[1] = __int_as_float(best_i); out[2] = z;
    }
}

__global__ void greedy_pick_kernel(const float* __restrict__ stats, int* __restrict__ out_token, float* __restrict__ out_logprob) {
    pdl_begin();
    const int row = blockIdx.x, lane = threadIdx.x;      // 32 threads, one chunk each
    const float* s = stats + ((size_t)row * GREEDY_CHUNKS + lane) * 3;
    float best = s[0];
    int best_i = __float_as_int(s[1]);
    const float m = best, z = s[2];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    float total = z == 0.f ? 0.f : z * expf(m - best);     // an empty chunk has max -inf and sum 0
    total = warp_sum(total);
    if (lane == 0) { out_token[row] = best_i; out_logprob[row] = -logf(total); }
}

// Greedy tokens and their log-probabilities (temperature 1) for `rows` rows; `stats` holds rows * 96 floats.
WLLM_API int wllm_sample_greedy(const float* logits, int row_stride, int rows, int V, float* stats, int* out_token,
                                float* out_logprob, cudaStream_t stream) {
    if (rows <= 0) return WLLM_OK;
    if (V <= 0 || row_stride < V) return WLLM_BAD_SIZE;
    const int st = wllm_launch(greedy_stats_kernel, dim3(GREEDY_CHUNKS, rows), 256, 0, stream, logits, row_stride, V, stats);
    if (st) return st;
    return wllm_launch(greedy_pick_kernel, rows, 32, 0, stream, (const float*)stats, out_token, out_logprob);
}

WLLM_API int wllm_sample(float* logits, int row_stride, int rows, int V, const float* temperature, const int* top_k,
                         const float* top_p, const float* min_p, const float* penalty, const int* seed_lo,
                         const int* seed_hi, const int* counter, const int* gen_offsets, const int* gen_ids,
                         int* out_token, float* out_logprob, cudaStream_t stream) {
    if (rows <= 0) return WLLM_OK;
    if (V <= 0 || row_stride < V) return WLLM_BAD_SIZE;
    return wllm_launch(sample_kernel, rows, THREADS, 0, stream, logits, row_stride, V, temperature, top_k, top_p, min_p, penalty,
                       seed_lo, seed_hi, counter, gen_offsets, gen_ids, out_token, out_logprob);
}
