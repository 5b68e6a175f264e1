// Gated feed-forward activation on a fused [gate | up] row:
//     out[n, c] = act(gate[n, c]) * up[n, c],   gate = in[n, c], up = in[n, I + c]
// evaluated in 32-bit and rounded once.  act 0: tanh-approximated GELU
//     0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)));  act 1: SiLU  x / (1 + exp(-x)).
#include "common.cuh"

__device__ __forceinline__ float act_gelu_tanh(float x) {
    const float k = 0.7978845608028654f;  // sqrt(2/pi)
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float act_silu(float x) { return x / (1.0f + expf(-x)); }

template <typename T, int ACT>
__global__ void gated_act_kernel(const T* __restrict__ in, T* __restrict__ out, int I, size_t total) {
    pdl_begin();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t n = idx / I, c = idx % I;
        const float g = to_f32(in[n * 2 * I + c]), u = to_f32(in[n * 2 * I + I + c]);
        out[idx] = from_f32<T>((ACT == 0 ? act_gelu_tanh(g) : act_silu(g)) * u);
    }
}

// bfloat16 rows whose width is a multiple of 8: 16-byte loads and stores, grid (column blocks, rows)
template <int ACT>
__global__ void gated_act_bf16x8_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int I) {
    pdl_begin();
    const int n = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= I) return;
    const uint4 gv = *reinterpret_cast<const uint4*>(in + (size_t)n * 2 * I + c);
    const uint4 uv = *reinterpret_cast<const uint4*>(in + (size_t)n * 2 * I + I + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
        o2[i] = __floats2bfloat162_rn((ACT == 0 ? act_gelu_tanh(g.x) : act_silu(g.x)) * u.x,
                                      (ACT == 0 ? act_gelu_tanh(g.y) : act_silu(g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + (size_t)n * I + c) = ov;
}

WLLM_API int wllm_gated_act(const void* in, void* out, int dtype, int act, int n, int I, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (I <= 0) return WLLM_BAD_SIZE;
    if (act != 0 && act != 1) return WLLM_BAD_SIZE;
    if (dtype == WLLM_BF16 && I % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const dim3 grid((I / 8 + 127) / 128, n);
        if (act == 0) return wllm_launch(gated_act_bf16x8_kernel<0>, grid, 128, 0, stream, (const bf16*)in, (bf16*)out, I);
        return wllm_launch(gated_act_bf16x8_kernel<1>, grid, 128, 0, stream, (const bf16*)in, (bf16*)out, I);
    }
    const size_t total = (size_t)n * I;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
#define LAUNCH(T, A) wllm_launch(gated_act_kernel<T, A>, blocks, threads, 0, stream, (const T*)in, (T*)out, I, total)
    if (dtype == WLLM_BF16) return act == 0 ? LAUNCH(bf16, 0) : LAUNCH(bf16, 1);
    if (dtype == WLLM_F32) return act == 0 ? LAUNCH(float, 0) : LAUNCH(float, 1);
#undef LAUNCH
    return WLLM_BAD_DTYPE;
}
