// True 32-bit matrix product  C[M, N] = A[M, K] * W[N, K]^T  on the FMA pipes.
//
// No tensor cores and no reduced-precision mode.  Every element of C is computed in one order, whatever
// kernel and tile it falls in:
//   segment   1,024 consecutive k that start at a multiple of 1,024: one chain of fused multiply-adds over
//             the segment's k in ascending order, starting from zero;
//   element   the segments' sums added one after the other in ascending order.
// A row of C therefore depends on its own row of A only, bit for bit, which makes the 32-bit path of the
// engine independent of batching.  (Zero padding past K adds fma(0, 0, acc) = acc.)
//
// Two kernels with that same arithmetic:
//   tile kernel    steps of many rows, bound by the FMA pipes: BM x 128 x 16 tiles (BM = 64 or 128), 256
//                  threads with 4 x 8 or 8 x 8 outputs each, operands transposed in shared memory and read
//                  as float4, the next tile fetched into registers while the current one is multiplied; the
//                  sums of finished segments wait in shared memory.
//   skinny kernel  steps of at most 32 rows, bound by streaming W once: a warp owns 32 rows of W and one
//                  segment (so a matrix of few rows and long K still gives every SM many warps), streams it
//                  through its own ring of cp.async stages and keeps one chain per row of A in each lane;
//                  a second kernel adds the segments' sums in order.
#include "common.cuh"

// ------------------------------------------------------------------------------------------------
// tile kernel
// ------------------------------------------------------------------------------------------------
constexpr int SEG = 1024;              // k per segment
constexpr int TBN = 128, TBK = 16;

template <int ROWS, bool VEC>
__device__ __forceinline__ void tile_fetch(const float* __restrict__ src, int ld, int rows, int K, int r0, int k0,
                                           int tid, float4 (&reg)[ROWS * 4 / 256]) {
    // ROWS rows x 16 k = ROWS * 4 groups of 4 along k
#pragma unroll
    for (int i = 0; i < ROWS * 4 / 256; ++i) {
        const int f = tid + i * 256;
        const int row = f >> 2, kq = (f & 3) * 4;
        const int gr = r0 + row, gk = k0 + kq;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (gr < rows) {
            const float* p = src + (size_t)gr * ld + gk;
            if (VEC) {
                if (gk < K) v = *reinterpret_cast<const float4*>(p);
            } else {
                if (gk < K) v.x = p[0];
                if (gk + 1 < K) v.y = p[1];
                if (gk + 2 < K) v.z = p[2];
                if (gk + 3 < K) v.w = p[3];
            }
        }
        reg[i] = v;
    }
}

template <int ROWS>
__device__ __forceinline__ void tile_stash(float (*dst)[ROWS + 4], int tid, const float4 (&reg)[ROWS * 4 / 256]) {
#pragma unroll
    for (int i = 0; i < ROWS * 4 / 256; ++i) {
        const int f = tid + i * 256;
        const int row = f >> 2, kq = (f & 3) * 4;
        dst[kq + 0][row] = reg[i].x;
        dst[kq + 1][row] = reg[i].y;
        dst[kq + 2][row] = reg[i].z;
        dst[kq + 3][row] = reg[i].w;
    }
}

template <int BM, bool VEC>
__global__ void __launch_bounds__(256, 2)
gemm_f32_tile_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw, float* __restrict__ C,
                     int ldc, int M, int N, int K) {
    constexpr int TM = BM / 16;            // 4 or 8 rows a thread: ty*4 + 0..3, and BM/2 + ty*4 + 0..3 when TM = 8
    __shared__ __align__(16) float As[2][TBK][BM + 4];
    __shared__ __align__(16) float Ws[2][TBK][TBN + 4];
    pdl_begin();
    const int tid = threadIdx.x;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * TBN;   // neighbours in the grid share a tile of W
    const int ty = tid >> 4, tx = tid & 15;
    extern __shared__ float totals[];      // [TM * 8][256]: the sum of the finished segments, when K has several
    float acc[TM][8];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    float4 ra[BM * 4 / 256], rw[TBN * 4 / 256];
    const int tiles = (K + TBK - 1) / TBK;
    tile_fetch<BM, VEC>(A, lda, M, K, m0, 0, tid, ra);
    tile_fetch<TBN, VEC>(W, ldw, N, K, n0, 0, tid, rw);
    tile_stash<BM>(As[0], tid, ra);
    tile_stash<TBN>(Ws[0], tid, rw);
    __syncthreads();
    for (int t = 0; t < tiles; ++t) {
        const int cur = t & 1;
        if (t + 1 < tiles) {
            tile_fetch<BM, VEC>(A, lda, M, K, m0, (t + 1) * TBK, tid, ra);
            tile_fetch<TBN, VEC>(W, ldw, N, K, n0, (t + 1) * TBK, tid, rw);
        }
#pragma unroll
        for (int k = 0; k < TBK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[cur][k][ty * 4]);
            const float4 a1 = TM == 8 ? *reinterpret_cast<const float4*>(&As[cur][k][BM / 2 + ty * 4]) : a0;
            const float4 b0 = *reinterpret_cast<const float4*>(&Ws[cur][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Ws[cur][k][TBN / 2 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (t + 1 < tiles) {
            tile_stash<BM>(As[cur ^ 1], tid, ra);
            tile_stash<TBN>(Ws[cur ^ 1], tid, rw);
            if (((t + 1) & (SEG / TBK - 1)) == 0) {     // a segment ends here and another follows
                const bool first = (t + 1) == SEG / TBK;
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float* tot = &totals[(i * 8 + j) * 256 + tid];
                        *tot = first ? acc[i][j] : *tot + acc[i][j];
                        acc[i][j] = 0.f;
                    }
            }
        }
        __syncthreads();
    }
    if (tiles > SEG / TBK) {
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] = totals[(i * 8 + j) * 256 + tid] + acc[i][j];
    }
    const bool vec_out = (ldc % 4 == 0) && ((uintptr_t)C % 16 == 0);
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + (i < 4 ? ty * 4 + i : BM / 2 + ty * 4 + (i - 4));
        if (gm >= M) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int gn = n0 + h * (TBN / 2) + tx * 4;
            float* dst = C + (size_t)gm * ldc + gn;
            if (vec_out && gn + 3 < N) {
                *reinterpret_cast<float4*>(dst) = make_float4(acc[i][h * 4], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (gn + j < N) dst[j] = acc[i][h * 4 + j];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// skinny kernel (K and the pitches in steps of 4 floats, 16-byte aligned operands)
// ------------------------------------------------------------------------------------------------
constexpr int SBN = 32, SBK = 32, SLD = SBK + 4;    // a warp's stage: 32 rows of 32 floats (128 contiguous bytes of W) + 4 of padding
constexpr int SWARPS = 4;
// Stages of a warp's ring.  Four (12 KB of W a warp ahead of its arithmetic, two CTAs an SM) is what a launch with
// tasks for every warp slot runs fastest with.  A launch of few tasks (the o projection of a 32-bit Gemma-7B step
// is 384 tasks for 148 SMs) lives on what each warp has in flight: it takes the deep ring, as deep as four warps'
// shared memory allows (28 KB a warp with up to 8 rows of A, 20 KB with 16; with 32 rows there is no room).
constexpr int SSTAGES_FULL = 4;
template <int BM> __host__ __device__ constexpr int skinny_deep_stages() { return BM <= 8 ? 8 : (BM <= 16 ? 6 : 4); }

__device__ __forceinline__ void cp_async_16(float* smem_dst, const float* src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;          // 0: the 16 bytes are filled with zeros, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A warp's task: rows n0..n0+31 of W, segment `seg`.  Lane x keeps BM chains, out[m][n0 + x], m < BM.
// `dst` is C when K has one segment, else the partial sums [segment][M][N].
template <int BM, int SSTAGES>
__global__ void __launch_bounds__(SWARPS * 32)
gemm_f32_skinny_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                       float* __restrict__ dst, int ld_dst, long long seg_stride, int M, int N, int K, int segs,
                       int tasks) {
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int task = blockIdx.x * SWARPS + warp;
    if (task >= tasks) return;
    float (*Ws)[SBN][SLD] = reinterpret_cast<float (*)[SBN][SLD]>(smem + (size_t)warp * SSTAGES * (SBN + BM) * SLD);
    float (*As)[BM][SLD] = reinterpret_cast<float (*)[BM][SLD]>(&Ws[SSTAGES][0][0]);
    const int n0 = (task / segs) * SBN, seg = task % segs;
    const int k_begin = seg * SEG, k_end = min(K, k_begin + SEG);
    const int tiles = (k_end - k_begin + SBK - 1) / SBK;

    auto issue_w = [&](int t, int stage) {        // 32 rows x 8 chunks of 16 bytes: an instruction takes 4 rows of 128 bytes
#pragma unroll
        for (int c = lane; c < SBN * (SBK / 4); c += 32) {
            const int row = c >> 3, gk = k_begin + t * SBK + (c & 7) * 4;
            const bool valid = n0 + row < N && gk < k_end;
            cp_async_16(&Ws[stage][row][(c & 7) * 4], valid ? W + (size_t)(n0 + row) * ldw + gk : W, valid);
        }
    };
    auto issue_a = [&](int t, int stage) {
#pragma unroll
        for (int c = lane; c < BM * (SBK / 4); c += 32) {
            const int row = c >> 3, gk = k_begin + t * SBK + (c & 7) * 4;
            const bool valid = row < M && gk < k_end;
            cp_async_16(&As[stage][row][(c & 7) * 4], valid ? A + (size_t)row * lda + gk : A, valid);
        }
    };
    // the weights are no kernel's output: their first stages are on the way before this kernel waits for the
    // kernel that writes A
#pragma unroll
    for (int s = 0; s < SSTAGES - 1; ++s)
        if (s < tiles) issue_w(s, s);
    pdl_wait();
#pragma unroll
    for (int s = 0; s < SSTAGES - 1; ++s) {
        if (s < tiles) issue_a(s, s);
        cp_async_commit();
    }
    float acc[BM];
#pragma unroll
    for (int i = 0; i < BM; ++i) acc[i] = 0.f;
    for (int t = 0; t < tiles; ++t) {
        cp_async_wait<SSTAGES - 2>();
        __syncwarp();                        // tile t has landed for every lane, and every lane is done with tile t-1
        const int ahead = t + SSTAGES - 1;
        if (ahead < tiles) {
            issue_w(ahead, ahead % SSTAGES);
            issue_a(ahead, ahead % SSTAGES);
        }
        cp_async_commit();
        const int st = t % SSTAGES;
#pragma unroll
        for (int kk = 0; kk < SBK; kk += 4) {
            const float4 w4 = *reinterpret_cast<const float4*>(&Ws[st][lane][kk]);
#pragma unroll
            for (int i = 0; i < BM; ++i) {
                const float4 a4 = *reinterpret_cast<const float4*>(&As[st][i][kk]);
                acc[i] = fmaf(a4.x, w4.x, acc[i]);
                acc[i] = fmaf(a4.y, w4.y, acc[i]);
                acc[i] = fmaf(a4.z, w4.z, acc[i]);
                acc[i] = fmaf(a4.w, w4.w, acc[i]);
            }
        }
    }
    cp_async_wait<0>();
    const int gn = n0 + lane;
    if (gn < N) {
        float* out = dst + (size_t)seg * seg_stride;
#pragma unroll
        for (int i = 0; i < BM; ++i)
            if (i < M) out[(size_t)i * ld_dst + gn] = acc[i];
    }
}

// C[m][n] = the segments' sums added in ascending order.
__global__ void __launch_bounds__(256)
gemm_f32_fold_kernel(const float* __restrict__ parts, float* __restrict__ C, int ldc, int M, int N, int segs) {
    pdl_begin();
    const size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= (size_t)M * N) return;
    float total = parts[idx];
    for (int s = 1; s < segs; ++s) total = total + parts[(size_t)s * M * N + idx];
    C[(idx / N) * ldc + idx % N] = total;
}

template <int BM, int STAGES>
static int launch_skinny_as(const float* A, int lda, const float* W, int ldw, float* C, int ldc, int M, int N, int K,
                            float* scratch, cudaStream_t stream) {
    const int segs = (K + SEG - 1) / SEG;
    const size_t smem = (size_t)SWARPS * STAGES * (SBN + BM) * SLD * sizeof(float);
    static bool raised = false;          // per instantiation; the attribute is a property of the function
    if (!raised) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_f32_skinny_kernel<BM, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)smem);
        if (e != cudaSuccess) return 1000 + (int)e;
        raised = true;
    }
    const int tasks = ((N + SBN - 1) / SBN) * segs;
    float* dst = segs > 1 ? scratch : C;
    const int st = wllm_launch(gemm_f32_skinny_kernel<BM, STAGES>, dim3((tasks + SWARPS - 1) / SWARPS), SWARPS * 32, smem, stream,
                               A, lda, W, ldw, dst, segs > 1 ? N : ldc, (long long)M * N, M, N, K, segs, tasks);
    if (st != WLLM_OK || segs == 1) return st;
    return wllm_launch(gemm_f32_fold_kernel, dim3((unsigned)(((size_t)M * N + 255) / 256)), 256, 0, stream,
                       (const float*)scratch, C, ldc, M, N, segs);
}

template <int BM>
static int launch_skinny(const float* A, int lda, const float* W, int ldw, float* C, int ldc, int M, int N, int K,
                         float* scratch, long long scratch_floats, cudaStream_t stream) {
    const int segs = (K + SEG - 1) / SEG;
    if (segs > 1 && (scratch == nullptr || scratch_floats < (long long)segs * M * N)) return WLLM_BAD_SIZE;
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            sms = 148;
    }
    const int tasks = ((N + SBN - 1) / SBN) * segs;
    constexpr int DEEP = skinny_deep_stages<BM>();
    if (DEEP != SSTAGES_FULL && tasks <= sms * SWARPS)      // at most one CTA's worth of warps an SM: few tasks
        return launch_skinny_as<BM, DEEP>(A, lda, W, ldw, C, ldc, M, N, K, scratch, stream);
    return launch_skinny_as<BM, SSTAGES_FULL>(A, lda, W, ldw, C, ldc, M, N, K, scratch, stream);
}

template <int BM, bool VEC>
static int launch_tile(const float* A, int lda, const float* W, int ldw, float* C, int ldc, int M, int N, int K,
                       cudaStream_t stream) {
    const size_t totals = K > SEG ? (size_t)(BM / 16) * 8 * 256 * sizeof(float) : 0;
    static bool raised = false;
    if (totals > 0 && !raised) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_f32_tile_kernel<BM, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)((size_t)(BM / 16) * 8 * 256 * sizeof(float)));
        if (e != cudaSuccess) return 1000 + (int)e;
        raised = true;
    }
    const dim3 grid((M + BM - 1) / BM, (N + TBN - 1) / TBN);
    return wllm_launch(gemm_f32_tile_kernel<BM, VEC>, grid, 256, totals, stream, A, lda, W, ldw, C, ldc, M, N, K);
}

// Floats of scratch that a product of these sizes needs (0: none): the skinny kernel's partial sums.
WLLM_API long long wllm_gemm_f32_scratch_floats(int M, int N, int K) {
    const int segs = (K + SEG - 1) / SEG;
    return (M <= 32 && segs > 1) ? (long long)segs * M * N : 0;
}

WLLM_API int wllm_gemm_f32(const float* A, int lda, const float* W, int ldw, float* C, int ldc, int M, int N, int K,
                           float* scratch, long long scratch_floats, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return WLLM_OK;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return WLLM_BAD_SIZE;
    const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
    if (vec && M <= 8) return launch_skinny<8>(A, lda, W, ldw, C, ldc, M, N, K, scratch, scratch_floats, stream);
    if (vec && M <= 16) return launch_skinny<16>(A, lda, W, ldw, C, ldc, M, N, K, scratch, scratch_floats, stream);
    if (vec && M <= 32) return launch_skinny<32>(A, lda, W, ldw, C, ldc, M, N, K, scratch, scratch_floats, stream);
    if (M <= 64) {
        if (vec) return launch_tile<64, true>(A, lda, W, ldw, C, ldc, M, N, K, stream);
        return launch_tile<64, false>(A, lda, W, ldw, C, ldc, M, N, K, stream);
    }
    if (vec) return launch_tile<128, true>(A, lda, W, ldw, C, ldc, M, N, K, stream);
    return launch_tile<128, false>(A, lda, W, ldw, C, ldc, M, N, K, stream);
}

// ------------------------------------------------------------------------------------------------
// What the FMA pipes give when nothing else is asked of them: the denominator of the products above.
// Every thread runs 8 independent chains of `iters` fused multiply-adds; out[blocks * 256] takes the sums.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) fma_loop_kernel(float* __restrict__ out, int iters, float a, float b) {
    float x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = (float)(threadIdx.x + j) * 1e-3f;
    for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = fmaf(x[j], a, b);
    }
    float total = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) total += x[j];
    out[(size_t)blockIdx.x * 256 + threadIdx.x] = total;
}

WLLM_API int wllm_fma_loop(float* out, int blocks, int iters, cudaStream_t stream) {
    if (blocks <= 0 || iters <= 0) return WLLM_BAD_SIZE;
    fma_loop_kernel<<<blocks, 256, 0, stream>>>(out, iters, 0.999f, 1e-4f);
    return wllm_launch_status();
}
