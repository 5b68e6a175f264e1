// Root-mean-square norm over the 32-bit residual stream, with the pending branch
// output folded in first:
//     r = resid[row] (+ delta[row]);  resid[row] = r  (when a delta is given);
//     out[i] = r * (1 / sqrt(mean(r^2) + eps)) * (offset + w)
// `delta` may come as `delta_splits` partial sums (slabs `delta_split_stride` elements apart, as the
// split-K matrix product leaves them); they are added in slab order.
// All arithmetic is 32-bit; `out` is rounded once to the matrix type.  With `rows`
// the kernel reads row rows[i] and writes row i (the final norm at the places whose
// logits are wanted) and leaves the residual untouched.  One block per row; the sum
// of squares is reduced in a fixed order that depends on nothing but the row.
#include "common.cuh"

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void load4<bf16>(const bf16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t*>(&a);
    t.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
}

// v += part 0 + part 1 + ... in that order.  The loads of sixteen parts are issued together (they do not
// depend on one another); only the additions are in sequence.
template <typename TD, int VEC>
__device__ __forceinline__ void add_parts(float (&v)[4], const TD* __restrict__ d, int parts, size_t stride) {
    if (parts == 1) {      // the common case: one tensor to add
        float dv[4] = {0.f, 0.f, 0.f, 0.f};
        if (VEC == 4) load4(d, dv); else dv[0] = to_f32(d[0]);
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[k] += dv[k];
        return;
    }
    for (int sp = 0; sp < parts; sp += 16) {
        float dv[16][4];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            dv[u][0] = dv[u][1] = dv[u][2] = dv[u][3] = 0.f;
            if (sp + u < parts) {
                if (VEC == 4) load4(d + (size_t)(sp + u) * stride, dv[u]);
                else dv[u][0] = to_f32(d[(size_t)(sp + u) * stride]);
            }
        }
#pragma unroll
        for (int u = 0; u < 16; ++u)
            if (sp + u < parts) {
#pragma unroll
                for (int k = 0; k < VEC; ++k) v[k] += dv[u][k];
            }
    }
}

// VEC = 4: rows whose width is a multiple of 4 are read and written four elements at a time.
// VPT = 1, 2 or 4: the whole row fits in registers with that many vectors a thread, and memory is passed
// over once; VPT = 0: wider rows (or VEC = 1) take two passes.
template <typename TD, typename TW, typename TO, int VEC, int VPT>
__global__ void rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta, int delta_splits,
                               size_t delta_split_stride, const TW* __restrict__ w, float eps, float offset,
                               TO* __restrict__ out, const int* __restrict__ rows, int H) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    constexpr bool one_pass = VEC == 4 && VPT > 0;
    constexpr int NV = VPT > 0 ? VPT : 1;
    float wv[NV][4];
    if (one_pass) {          // the gain is written by no kernel: it is read while the predecessor still runs
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = (threadIdx.x + k * blockDim.x) * 4;
            wv[k][0] = wv[k][1] = wv[k][2] = wv[k][3] = 0.f;
            if (c < H) load4(w + c, wv[k]);
        }
    }
    pdl_wait();
    const int i = blockIdx.x;
    const int row = rows ? rows[i] : i;
    float* r = resid + (size_t)row * H;
    const TD* d = delta ? delta + (size_t)row * H : nullptr;
    const bool write_back = (d != nullptr) && (rows == nullptr);
    TO* o = out + (size_t)i * H;
    if (one_pass) {
        float v[NV][4];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = (threadIdx.x + k * blockDim.x) * 4;
            v[k][0] = v[k][1] = v[k][2] = v[k][3] = 0.f;
            if (c < H) {
                load4(r + c, v[k]);
                if (d) add_parts<TD, 4>(v[k], d + c, delta_splits, delta_split_stride);
#pragma unroll
                for (int e = 0; e < 4; ++e) ss += v[k][e] * v[k][e];
            }
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = (threadIdx.x + k * blockDim.x) * 4;
            if (c < H) {
                float y[4];
                if (write_back) store4(r + c, v[k]);
#pragma unroll
                for (int e = 0; e < 4; ++e) y[e] = (v[k][e] * inv) * (offset + wv[k][e]);
                store4(o + c, y);
            }
        }
        return;
    }
    float ss = 0.f;
    for (int c = threadIdx.x * VEC; c < H; c += blockDim.x * VEC) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (VEC == 4) load4(r + c, v); else v[0] = r[c];
        if (d) add_parts<TD, VEC>(v, d + c, delta_splits, delta_split_stride);
#pragma unroll
        for (int k = 0; k < VEC; ++k) ss += v[k] * v[k];
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x * VEC; c < H; c += blockDim.x * VEC) {
        float v[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
        if (VEC == 4) { load4(r + c, v); load4(w + c, wv); }
        else { v[0] = r[c]; wv[0] = to_f32(w[c]); }
        if (d) add_parts<TD, VEC>(v, d + c, delta_splits, delta_split_stride);
        if (write_back) {
            if (VEC == 4) store4(r + c, v); else r[c] = v[0];
        }
        float y[4];
#pragma unroll
        for (int k = 0; k < VEC; ++k) y[k] = (v[k] * inv) * (offset + wv[k]);
        if (VEC == 4) store4(o + c, y); else o[c] = from_f32<TO>(y[0]);
    }
}

template <typename TD, typename TW>
static int launch_out(float* resid, const void* delta, int delta_splits, size_t delta_split_stride, const void* w, float eps,
                      float offset, void* out, int out_dtype, const int* rows, int n, int H, cudaStream_t stream) {
    const bool vec = H % 4 == 0 && ((uintptr_t)resid & 15) == 0 && ((uintptr_t)delta & 15) == 0 &&
                     ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0 && delta_split_stride % 4 == 0;
    const int per = vec ? 4 : 1;
    const int threads = H / per >= 512 ? 512 : (H / per >= 256 ? 256 : 128);   // one vector a thread up to 2048 columns
    const int vpt = !vec ? 0 : (H <= threads * 4 ? 1 : (H <= threads * 8 ? 2 : (H <= threads * 16 ? 4 : 0)));
#define GO(TO, V, P) wllm_launch(rmsnorm_kernel<TD, TW, TO, V, P>, n, threads, 0, stream, resid, (const TD*)delta, delta_splits, \
                       delta_split_stride, (const TW*)w, eps, offset, (TO*)out, rows, H)
#define PICK(TO) (vpt == 1 ? GO(TO, 4, 1) : vpt == 2 ? GO(TO, 4, 2) : vpt == 4 ? GO(TO, 4, 4) : vec ? GO(TO, 4, 0) : GO(TO, 1, 0))
    if (out_dtype == WLLM_BF16) return PICK(bf16);
    if (out_dtype == WLLM_F32) return PICK(float);
#undef PICK
#undef GO
    return WLLM_BAD_DTYPE;
}

WLLM_API int wllm_rmsnorm(float* resid, const void* delta, int delta_dtype, int delta_splits, long long delta_split_stride,
                          const void* w, int w_dtype, float eps, float offset, void* out, int out_dtype, const int* rows,
                          int n, int H, cudaStream_t stream) {
    if (n <= 0) return WLLM_OK;
    if (H <= 0 || delta_splits < 1 || delta_split_stride < 0) return WLLM_BAD_SIZE;
    const bool dbf = delta_dtype == WLLM_BF16, wbf = w_dtype == WLLM_BF16;
    if ((delta_dtype != WLLM_BF16 && delta_dtype != WLLM_F32) || (w_dtype != WLLM_BF16 && w_dtype != WLLM_F32)) return WLLM_BAD_DTYPE;
    if (dbf && wbf) return launch_out<bf16, bf16>(resid, delta, delta_splits, (size_t)delta_split_stride, w, eps, offset, out, out_dtype, rows, n, H, stream);
    if (dbf && !wbf) return launch_out<bf16, float>(resid, delta, delta_splits, (size_t)delta_split_stride, w, eps, offset, out, out_dtype, rows, n, H, stream);
    if (!dbf && wbf) return launch_out<float, bf16>(resid, delta, delta_splits, (size_t)delta_split_stride, w, eps, offset, out, out_dtype, rows, n, H, stream);
    return launch_out<float, float>(resid, delta, delta_splits, (size_t)delta_split_stride, w, eps, offset, out, out_dtype, rows, n, H, stream);
}
