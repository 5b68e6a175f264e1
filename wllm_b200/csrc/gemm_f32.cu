// True 32-bit matrix product  C[M, N] = A[M, K] * W[N, K]^T  on the FMA pipes.
//
// No tensor cores, no reduced-precision mode, no split along K: every element of C
// is one chain of fused multiply-adds over k = 0..K-1 in ascending order, whatever
// tile it falls in.  A row of C therefore depends on its own row of A only, bit for
// bit, which makes the 32-bit path of the engine independent of batching.
// 128x128x16 tiles, 256 threads, 8x8 outputs per thread.
#include "common.cuh"

constexpr int BM = 128, BN = 128, BK = 16, TM = 8, TN = 8;

template <bool VEC>
__device__ __forceinline__ void load_tile(const float* __restrict__ src, int ld, int rows, int K, int r0, int k0,
                                          float (*dst)[BM + 4], int tid) {
    // 128 rows x 16 k = 512 groups of 4 along k; 2 groups per thread
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int f = tid + i * 256;
        const int row = f >> 2, kq = (f & 3) * 4;
        const int gr = r0 + row, gk = k0 + kq;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (gr < rows) {
            const float* p = src + (size_t)gr * ld + gk;
            if (VEC) {
                if (gk < K) {
                    const float4 t = *reinterpret_cast<const float4*>(p);
                    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
                }
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (gk + c < K) v[c] = p[c];
            }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) dst[kq + c][row] = v[c];
    }
}

template <bool VEC>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw, float* __restrict__ C,
                int ldc, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_begin();
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int ty = tid >> 4, tx = tid & 15;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        load_tile<VEC>(A, lda, M, K, m0, k0, As, tid);
        load_tile<VEC>(W, ldw, N, K, n0, k0, Ws, tid);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
        }
    }
}

WLLM_API int wllm_gemm_f32(const float* A, int lda, const float* W, int ldw, float* C, int ldc, int M, int N, int K,
                           cudaStream_t stream) {
    if (M <= 0 || N <= 0) return WLLM_OK;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return WLLM_BAD_SIZE;
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
    if (vec) return wllm_launch(gemm_f32_kernel<true>, grid, 256, 0, stream, A, lda, W, ldw, C, ldc, M, N, K);
    return wllm_launch(gemm_f32_kernel<false>, grid, 256, 0, stream, A, lda, W, ldw, C, ldc, M, N, K);
}
