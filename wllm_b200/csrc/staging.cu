// Host-side helpers for the small copies around a step: no kernels, only the runtime calls that move a
// step's index arrays to the device and its sampled ids back, each sequence behind one C entry point so
// that the host pays for one call instead of a dozen trips through a Python binding.
//
//   wllm_stage_send     pinned host -> device staging buffer on a copy stream, then staging -> destination
//                       on the step's stream, with the events that order the two streams;
//   wllm_stage_fetch    device -> pinned host on a copy stream, behind what the step's stream has queued.
//
// Events are made once by the caller's ring (wllm_event_create) and reused; they carry no timing.
#include "common.cuh"

static inline int status_of(cudaError_t e) { return e == cudaSuccess ? WLLM_OK : 1000 + (int)e; }

WLLM_API int wllm_event_create(void** out) {
    cudaEvent_t ev = nullptr;
    const cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    *out = (void*)ev;
    return status_of(e);
}

WLLM_API int wllm_event_destroy(void* event) {
    return event ? status_of(cudaEventDestroy((cudaEvent_t)event)) : WLLM_OK;
}

// Blocks the host until the work recorded in `event` is done.
WLLM_API int wllm_event_wait(void* event) { return status_of(cudaEventSynchronize((cudaEvent_t)event)); }

// `bytes` from `pinned` to `dst`, by way of `staged`:
//   copy stream: waits for `consumed` when `wait_consumed` is set (the staging buffer's last reader), copies
//                pinned -> staged, records `arrived`;
//   step stream: waits for `arrived`, copies staged -> dst, records `consumed`.
// The pinned buffer may be written again once `arrived` is done, the staging buffer once `consumed` is.
WLLM_API int wllm_stage_send(const void* pinned, void* staged, void* dst, long long bytes, cudaStream_t copy_stream,
                             cudaStream_t step_stream, void* arrived, void* consumed, int wait_consumed) {
    if (bytes <= 0) return WLLM_OK;
    cudaError_t e = cudaSuccess;
    if (wait_consumed) e = cudaStreamWaitEvent(copy_stream, (cudaEvent_t)consumed, 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(staged, pinned, (size_t)bytes, cudaMemcpyHostToDevice, copy_stream);
    if (e == cudaSuccess) e = cudaEventRecord((cudaEvent_t)arrived, copy_stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(step_stream, (cudaEvent_t)arrived, 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dst, staged, (size_t)bytes, cudaMemcpyDeviceToDevice, step_stream);
    if (e == cudaSuccess) e = cudaEventRecord((cudaEvent_t)consumed, step_stream);
    return status_of(e);
}

// `bytes` from `src` (device) to `pinned`, on the copy stream, behind everything the step's stream holds now:
// `queued` is recorded on the step's stream and awaited by the copy stream; `done` is recorded behind the copy.
// `extra_bytes` from `extra` (device; the kernels' status word) land right behind them in `pinned`.
WLLM_API int wllm_stage_fetch(void* pinned, const void* src, long long bytes, const void* extra, long long extra_bytes,
                              cudaStream_t step_stream, cudaStream_t copy_stream, void* queued, void* done) {
    if (bytes <= 0) return WLLM_OK;
    cudaError_t e = cudaEventRecord((cudaEvent_t)queued, step_stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(copy_stream, (cudaEvent_t)queued, 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(pinned, src, (size_t)bytes, cudaMemcpyDeviceToHost, copy_stream);
    if (e == cudaSuccess && extra != nullptr && extra_bytes > 0)
        e = cudaMemcpyAsync((char*)pinned + bytes, extra, (size_t)extra_bytes, cudaMemcpyDeviceToHost, copy_stream);
    if (e == cudaSuccess) e = cudaEventRecord((cudaEvent_t)done, copy_stream);
    return status_of(e);
}

// The step's stream waits for `event` (recorded on another stream).
WLLM_API int wllm_stream_wait(cudaStream_t stream, void* event) {
    return status_of(cudaStreamWaitEvent(stream, (cudaEvent_t)event, 0));
}
