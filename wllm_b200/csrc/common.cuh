// Shared by every kernel family: element types, status codes, reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define WLLM_API extern "C" __attribute__((visibility("default")))

// Status codes returned by every entry point (0 = launched).  Values of 1000 and
// above are 1000 + the cudaError_t of the failed launch.
#define WLLM_OK 0
#define WLLM_BAD_DTYPE 1
#define WLLM_BAD_SIZE 2
#define WLLM_BAD_ALIGN 3

// Element types as the Python side names them.
#define WLLM_F32 0
#define WLLM_BF16 1

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// One rotary pair turned by the angle whose sine and cosine are given: every product and sum rounded on its own
// (no contraction that one kernel's compilation might make and another's not), so that every kernel that rotates
// gives the same bits.
__device__ __forceinline__ void rotate_pair(float x1, float x2, float sn, float cs, float& y1, float& y2) {
    y1 = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
    y2 = __fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn));
}

static inline int wllm_launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? WLLM_OK : 1000 + (int)e;
}

// Programmatic dependent launch.  Every kernel of the engine begins with pdl_begin(): it lets the kernel
// behind it in the stream be scheduled at once (launch_dependents), then waits until the kernel before it
// has completed and its writes are visible (wait).  What a kernel does before its wait may touch shared
// memory and read-only inputs that no kernel of the step writes (weights), nothing else.  Launched with
// the attribute below, the launch latency and prologue of a kernel overlap the tail of its predecessor;
// without it (WLLM_PDL=0) both instructions do nothing and the stream serialises as usual.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_begin() { pdl_launch_dependents(); pdl_wait(); }

static inline bool wllm_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("WLLM_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on != 0;
}

template <typename... KArgs, typename... Args>
static inline int wllm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = wllm_pdl_enabled() ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    return e == cudaSuccess ? WLLM_OK : 1000 + (int)e;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block in a fixed order: xor tree inside each warp, then every thread
// adds the warps' partial sums in warp order.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];
    return total;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    v = warp_max(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = -INFINITY;
    for (int w = 0; w < nwarps; ++w) total = fmaxf(total, scratch[w]);
    return total;
}
