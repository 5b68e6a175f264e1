// Root-mean-square norm over the 32-bit residual stream, with the pending branch
// output folded in first:
//     r = resid[row] (+ delta[row]);  resid[row] = r  (when a delta is given);
//     out[i] = r * (1 / sqrt(mean(r^2) + eps)) * (offset + w)
// All arithmetic is 32-bit; `out` is rounded once to the matrix type.  With `rows`
// the kernel reads row rows[i] and writes row i (the final norm at the places whose
// logits are wanted) and leaves the residual untouched.  One block per row; the sum
// of squares is reduced in a fixed order that depends on nothing but the row.
#include "common.cuh"

template <typename TD, typename TW, typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta, const TW* __restrict__ w,
                               float eps, float offset, TO* __restrict__ out, const int* __restrict__ rows, int H) {
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const int row = rows ? rows[i] : i;
    float* r = resid + (size_t)row * H;
    const TD* d = delta ? delta + (size_t)row * H : nullptr;
    const bool write_back = (d != nullptr) && (rows == nullptr);
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = r[c];
        if (d) v += to_f32(d[c]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)i * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = r[c];
        if (d) v += to_f32(d[c]);
        if (write_back) r[c] = v;
        o[c] = from_f32<TO>((v * inv) * (offset + to_f32(w[c])));
    }
}

template <typename TD, typename TW>
static int launch_out(float* resid, const void* delta, const void* w, float eps, float offset, void* out, int out_dtype,
                      const int* rows, int n, int H, cudaStream_t stream) {
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (out_dtype == WLLM_BF16)
        rmsnorm_kernel<TD, TW, bf16><<<n, threads, 0, stream>>>(resid, (const TD*)delta, (const TW*)w, eps, offset, (bf16*)out, rows, H);
    else if (out_dtype == WLLM_F32)
        rmsnorm_kernel<TD, TW, float><<<n, threads, 0, stream>>>(resid, (const TD*)delta, (const TW*)w, eps, offset, (float*)out, rows, H);
    else
        return WLLM_BAD_DTYPE;
    return wllm_launch_status();
}

WLLM_API int wllm_rmsnorm(float* resid, const void* delta, int delta_dtype, const void* w, int w_dtype, float eps,
                          float offset, void* out, int out_dtype, const int* rows, int n, int H, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (H <= 0) return WLLM_BAD_SIZE;
    const bool dbf = delta_dtype == WLLM_BF16, wbf = w_dtype == WLLM_BF16;
    if ((delta_dtype != WLLM_BF16 && delta_dtype != WLLM_F32) || (w_dtype != WLLM_BF16 && w_dtype != WLLM_F32)) return WLLM_BAD_DTYPE;
    if (dbf && wbf) return launch_out<bf16, bf16>(resid, delta, w, eps, offset, out, out_dtype, rows, n, H, stream);
    if (dbf && !wbf) return launch_out<bf16, float>(resid, delta, w, eps, offset, out, out_dtype, rows, n, H, stream);
    if (!dbf && wbf) return launch_out<float, bf16>(resid, delta, w, eps, offset, out, out_dtype, rows, n, H, stream);
    return launch_out<float, float>(resid, delta, w, eps, offset, out, out_dtype, rows, n, H, stream);
}
