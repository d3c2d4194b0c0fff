// Building blocks of the weight-streaming kernels: 1-D TMA bulk copies into a
// shared-memory ring guarded by mbarriers, programmatic dependent launch, and the
// per-row dot product against activations staged in shared memory.
//
// Decode-time linear layers are pure HBM streaming: a weight matrix of a few MB is
// read once per token.  Rows of a packed matrix are contiguous, so a tile of R rows
// is one contiguous byte range and is fetched with a single cp.async.bulk; a ring of
// stages keeps tens of KB in flight per SM independently of how the math is mapped
// to lanes.  Every wait on an mbarrier is bounded: when the bound is hit the kernel
// raises a status word, drains its own copies and returns.
#pragma once

#include "linear.cuh"

namespace b200 {

// Host-visible status word of the streaming kernels (0 = ok, 1 = a bounded wait ran
// out).  Device pointer; allocated on first use.
int* stream_status_ptr();
int stream_status_check(const char* who);   // reads the word back (synchronises)

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait (each try_wait already sleeps for a hardware-defined interval).
constexpr uint32_t MBAR_SPIN_LIMIT = 1u << 22;
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, int* status, uint32_t limit) {
    for (uint32_t it = 0; it < limit; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(status, 1);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status) {
    return mbar_wait_limit(bar, parity, status, MBAR_SPIN_LIMIT);
}
// Contiguous global -> shared copy through the TMA unit; src, dst 16-byte aligned,
// bytes a multiple of 16.  Completion is counted on `bar` (no multicast).
__device__ __forceinline__ void tma_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Programmatic dependent launch: let the next kernel in the stream start its
// prologue (it only prefetches weights before its own pdl_wait), and wait for the
// previous kernel's results.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- activations in shared memory -------------------------------------------
// x is stored "unit-major": the 32 activations a 32-weight unit multiplies are
// contiguous, units are 36 floats apart so that eight lanes reading eight different
// units with 128-bit loads touch 32 distinct banks.
constexpr int XU_STRIDE = 36;
__host__ __device__ inline int xs_floats(int K) { return (K >> 5) * XU_STRIDE; }

template <int KIND>
__device__ __forceinline__ int xs_index(int k) {
    if (KIND == 3) {
        const int sb = k >> 8, r = k & 255;
        const int u = sb * 8 + (r >> 6) * 2 + ((r >> 4) & 1);
        return u * XU_STRIDE + ((r >> 5) & 1) * 16 + (r & 15);
    }
    return (k >> 5) * XU_STRIDE + (k & 31);
}

// Dot products of one weight row (in shared or global memory) with M (<= MT)
// activation vectors laid out by xs_index; returns full sums in every lane.
template <int KIND, int MT>
__device__ __forceinline__ void row_dot_xs(const uint8_t* row, const float* xs, int xs_tok_stride, int M,
                                           int K, int lane, float (&acc)[MT]) {
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
    const int U = K >> 5;
    for (int u = lane; u < U; u += 32) {
        float wv[32];
        if constexpr (KIND <= 3) load_unit<KIND, false>(row, u, wv);
        else load_unit_plain_generic<KIND>(row, u, wv);
        const float* xu = xs + u * XU_STRIDE;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                const float4* xp = reinterpret_cast<const float4*>(xu + m * xs_tok_stride);
                float s = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 a = xp[i];
                    s += a.x * wv[4 * i] + a.y * wv[4 * i + 1] + a.z * wv[4 * i + 2] + a.w * wv[4 * i + 3];
                }
                acc[m] += s;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = warp_sum(acc[m]);
}
#endif

}  // namespace b200
