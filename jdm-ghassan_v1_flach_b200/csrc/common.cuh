// Shared host/device plumbing of the b200ops library: status codes, the current
// stream, grow-only device workspaces, and small device helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/b200ops.h"

namespace b200 {

// ---- status ---------------------------------------------------------------
int fail(int code, const char* fmt, ...);      // records the message, returns code
int cuda_status(cudaError_t e, const char* what);
cudaStream_t stream();
extern unsigned long long g_kernel_launches;   // kernels enqueued by this library so far

#define B200_REQUIRE(cond, ...)                                 \
    do {                                                        \
        if (!(cond)) return b200::fail(B200_EINVAL, __VA_ARGS__); \
    } while (0)

#define B200_CUDA(call)                                              \
    do {                                                             \
        cudaError_t e__ = (call);                                    \
        if (e__ != cudaSuccess) return b200::cuda_status(e__, #call); \
    } while (0)

// Checked after every launch, like the reference's cudaGetLastError() checks.
#define B200_LAUNCH_CHECK(name)                                           \
    do {                                                                  \
        cudaError_t e__ = cudaGetLastError();                             \
        if (e__ != cudaSuccess) return b200::cuda_status(e__, name);      \
        ++b200::g_kernel_launches;                                        \
    } while (0)

// ---- workspaces -----------------------------------------------------------
// Grow-only cached device buffers (rounded up to 1 MiB).  Growth calls
// cudaMalloc, which synchronises the device: reserve before a stream capture.
struct Workspace {
    void* ptr = nullptr;
    size_t bytes = 0;
    int ensure(size_t need, void** out);
    void release();
};
enum { WS_LINEAR = 0, WS_MOE = 1, WS_MAMBA = 2, WS_ATTN = 3, WS_SAMPLE = 4, WS_PERM = 5, WS_ROUTE = 6, WS_PREFILL = 7, WS_SPLITK = 8, WS_COUNT = 9 };
Workspace& workspace(int which);
unsigned long long workspace_generation();   // changes whenever a workspace address goes stale

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
int num_sms();
// Second stream for work independent of the current stream's (see runtime.cu): between
// side_begin() and side_end() stream() is the side stream; side_wait() joins.
// Named ranges for timeline tools (NVTX; a no-op without a tool attached).
void nvtx_push(const char* name);
void nvtx_pop();
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtx_push(name); }
    ~NvtxRange() { nvtx_pop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};
int side_begin();
int side_end();
int side_wait();

// Status word of the kernels with bounded waits (0 = ok).  Device pointer, allocated
// on first use; the check reads it back (synchronising copy) and clears it.
int* stream_status_ptr();
int stream_status_check(const char* who);

// ---- device helpers -------------------------------------------------------
#ifdef __CUDACC__
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
// Block-wide sum; `red` is shared memory for at least 32 floats.  All threads get
// the result.  Safe to call repeatedly (leading barrier protects `red`).
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double block_sum_d(double v, double* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = warp_sum_d(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    double t = (lane < nw) ? red[lane] : 0.0;
    t = warp_sum_d(t);
    return t;
}
__device__ __forceinline__ float half_bits_to_float(uint16_t h) {
    return __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ uint16_t float_to_half_bits(float f) {
    return __half_as_ushort(__float2half_rn(f));
}
// x / (1 + exp(-x)) with the accurate expf, as the reference CPU path computes it.
__device__ __forceinline__ float silu_acc(float v) { return v / (1.0f + expf(-v)); }
#endif

}  // namespace b200
