// Shared pieces of the row-streaming linear kernels: the weight-kind tags, the
// per-row dot product every GEMV-shaped kernel (plain linear, Mamba projections,
// MoE experts) is built from, and the host entry points.
#pragma once

#include <algorithm>

#include "quant.cuh"

namespace b200 {

// Template tags for unpacked weights, next to the packed kinds 0..3.
constexpr int KIND_F16 = 4;
constexpr int KIND_F32 = 5;

// Public "qkind" (-1 fp16, 0..3 packed) -> template tag.
static inline int tag_of_qkind(int qkind) { return qkind < 0 ? KIND_F16 : qkind; }

__host__ __device__ inline int64_t row_bytes_of(int kind, int K) {
    if (kind == KIND_F16) return (int64_t)K * 2;
    if (kind == KIND_F32) return (int64_t)K * 4;
    return q_row_bytes(kind, K);
}

constexpr int GEMV_WARPS = 4;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;

struct GemvArgs {
    const float* x;     // [M,K]
    const uint8_t* w;   // [N,K] in the kernel's weight kind
    float* y;           // [M,N]
    int M, K, N;
};

int linear(const float* x, const void* w, int kind, float* y, int M, int K, int N);
// True when linear() would take the tensor-core GEMM for this call; linear_a16() then runs that
// GEMM straight from fp16 rows a16 [M, K] (the producer rounded them, as pack_rows_f16 would).
bool linear_uses_gemm(const void* w, int kind, const float* y, int M, int K, int N);
int linear_a16(const void* a16, const void* w, int kind, float* y, int M, int K, int N);
int dequantize(const uint8_t* src, uint16_t* dst, int64_t n, int kind);

#ifdef __CUDACC__
// 32 consecutive weights of an unpacked row.
template <int KIND>
__device__ __forceinline__ void load_unit_plain(const uint8_t* row, int u, float (&w)[32]) {
    if (KIND == KIND_F16) {
        const uint4* p = reinterpret_cast<const uint4*>(row) + (int64_t)u * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 v = __ldg(p + i);
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&words[j]));
                w[8 * i + 2 * j] = f.x;
                w[8 * i + 2 * j + 1] = f.y;
            }
        }
    } else {
        const float4* p = reinterpret_cast<const float4*>(row) + (int64_t)u * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 v = __ldg(p + i);
            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
        }
    }
}

// Same through generic loads (the row may live in shared memory).
template <int KIND>
__device__ __forceinline__ void load_unit_plain_generic(const uint8_t* row, int u, float (&w)[32]) {
    if (KIND == KIND_F16) {
        const uint4* p = reinterpret_cast<const uint4*>(row) + (int64_t)u * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 v = p[i];
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&words[j]));
                w[8 * i + 2 * j] = f.x;
                w[8 * i + 2 * j + 1] = f.y;
            }
        }
    } else {
        const float4* p = reinterpret_cast<const float4*>(row) + (int64_t)u * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 v = p[i];
            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
        }
    }
}

// Dot products of weight row n with M (<= MT) activation rows.  Lanes split the
// row's 32-weight units; on return every lane holds the full sums.  Packed weights
// enter with their exact dequantised fp32 value, as in the reference's fused CUDA
// kernel (cuda/kernels.cu:549-598); its CPU path rounds each value through fp16
// first (core/ops.cpp:392), a 2^-12 relative perturbation per weight.
// Requires K % 32 == 0 and x 16-byte aligned.
template <int KIND, int MT>
__device__ __forceinline__ void gemv_row(const float* __restrict__ x, const uint8_t* __restrict__ w,
                                         int64_t n, int M, int K, int lane, float (&acc)[MT]) {
    const uint8_t* row = w + n * row_bytes_of(KIND, K);
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
    const int U = K >> 5;
    for (int u = lane; u < U; u += 32) {
        float wv[32];
        int k_lo, k_hi;
        if constexpr (KIND <= 3) {
            load_unit<KIND, false>(row, u, wv);
            unit_k<KIND>(u, k_lo, k_hi);
        } else {
            load_unit_plain<KIND>(row, u, wv);
            k_lo = u * 32;
            k_hi = k_lo + 16;
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                const float4* xa = reinterpret_cast<const float4*>(x + (int64_t)m * K + k_lo);
                const float4* xb = reinterpret_cast<const float4*>(x + (int64_t)m * K + k_hi);
                float s = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 a = __ldg(xa + i);
                    s += a.x * wv[4 * i] + a.y * wv[4 * i + 1] + a.z * wv[4 * i + 2] + a.w * wv[4 * i + 3];
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 b = __ldg(xb + i);
                    s += b.x * wv[16 + 4 * i] + b.y * wv[17 + 4 * i] + b.z * wv[18 + 4 * i] + b.w * wv[19 + 4 * i];
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
