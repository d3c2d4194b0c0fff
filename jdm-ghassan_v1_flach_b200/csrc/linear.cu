// Linear layers over fp32 / fp16 / packed weights, the materialising dequantiser
// and the small layout ops that sit beside them.
//
// y[M,N] = x[M,K] . W^T with W row-major [N,K] (reference: cpu::linear_forward,
// core/math_cpu.cpp:117-134; ops::linear_forward_q4, core/ops.cpp:360-401; CUDA
// side cuda/kernels.cu:482-633).
//
// Decode shapes (M <= 8) are HBM-bound weight streaming: one warp per output row,
// each lane dequantises 32-weight units in registers and the row sum is a warp
// shuffle reduction; every token of the tile reuses the registers.  Larger M walks
// the same kernel over token tiles of 8 (weights then come from L2).
#include "fused.cuh"
#include "gemm.cuh"

namespace b200 {

// ---------------------------------------------------------------------------
// dequantize_quant: packed -> fp16, bit-exact with ops::quant_materialize on CPU.
// ---------------------------------------------------------------------------
template <int KIND>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ src,
                                                      uint16_t* __restrict__ dst, int64_t n) {
    const int64_t groups = (n + 7) / 8;
    for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < groups;
         g += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i0 = g * 8;
        if (i0 + 8 <= n) {
            uint32_t out[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t lo = float_to_half_bits(q_value<KIND>(src, i0 + 2 * j));
                const uint32_t hi = float_to_half_bits(q_value<KIND>(src, i0 + 2 * j + 1));
                out[j] = lo | (hi << 16);
            }
            *reinterpret_cast<uint4*>(dst + i0) = make_uint4(out[0], out[1], out[2], out[3]);
        } else {
            for (int64_t i = i0; i < n; ++i) dst[i] = float_to_half_bits(q_value<KIND>(src, i));
        }
    }
}

int dequantize(const uint8_t* src, uint16_t* dst, int64_t n, int kind) {
    B200_REQUIRE(src && dst && n > 0, "dequantize_quant: bad arguments");
    B200_REQUIRE(kind >= 0 && kind <= 3, "dequantize_quant: unknown kind %d", kind);
    B200_REQUIRE((reinterpret_cast<uintptr_t>(dst) & 15) == 0, "dequantize_quant: dst must be 16-byte aligned");
    const int64_t groups = (n + 7) / 8;
    const int grid = (int)std::min<int64_t>(ceil_div64(groups, 256), (int64_t)num_sms() * 32);
    switch (kind) {
        case 0: dequant_kernel<0><<<grid, 256, 0, stream()>>>(src, dst, n); break;
        case 1: dequant_kernel<1><<<grid, 256, 0, stream()>>>(src, dst, n); break;
        case 2: dequant_kernel<2><<<grid, 256, 0, stream()>>>(src, dst, n); break;
        default: dequant_kernel<3><<<grid, 256, 0, stream()>>>(src, dst, n); break;
    }
    B200_LAUNCH_CHECK("dequant_kernel");
    return B200_OK;
}

// ---------------------------------------------------------------------------
// Row-streaming GEMV (M <= MT tokens per pass).
// ---------------------------------------------------------------------------
template <int KIND, int MT>
__global__ void __launch_bounds__(GEMV_THREADS) gemv_kernel(GemvArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * GEMV_WARPS + warp;
    if (n >= a.N) return;
    float acc[MT];
    gemv_row<KIND, MT>(a.x, a.w, n, a.M, a.K, lane, acc);
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m)
            if (m < a.M) a.y[(int64_t)m * a.N + n] = acc[m];
    }
}

// Slow but general: K not a multiple of 32 (fp32 / fp16 weights only).
template <int KIND>
__global__ void __launch_bounds__(128) gemv_ragged_kernel(GemvArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 4 + warp;
    if (n >= a.N) return;
    for (int m = 0; m < a.M; ++m) {
        float acc = 0.0f;
        for (int k = lane; k < a.K; k += 32) {
            const float wv = KIND == KIND_F32
                                 ? reinterpret_cast<const float*>(a.w)[(int64_t)n * a.K + k]
                                 : half_bits_to_float(reinterpret_cast<const uint16_t*>(a.w)[(int64_t)n * a.K + k]);
            acc += a.x[(int64_t)m * a.K + k] * wv;
        }
        acc = warp_sum(acc);
        if (lane == 0) a.y[(int64_t)m * a.N + n] = acc;
    }
}

template <int KIND>
static int launch_gemv_kind(const GemvArgs& a) {
    const int grid = ceil_div(a.N, GEMV_WARPS);
    if (a.M == 1) gemv_kernel<KIND, 1><<<grid, GEMV_THREADS, 0, stream()>>>(a);
    else if (a.M == 2) gemv_kernel<KIND, 2><<<grid, GEMV_THREADS, 0, stream()>>>(a);
    else if (a.M <= 4) gemv_kernel<KIND, 4><<<grid, GEMV_THREADS, 0, stream()>>>(a);
    else gemv_kernel<KIND, 8><<<grid, GEMV_THREADS, 0, stream()>>>(a);
    B200_LAUNCH_CHECK("gemv_kernel");
    return B200_OK;
}

// kind: KIND_F32 / KIND_F16 / 0..3.  Any M; tokens are processed 8 at a time.
bool linear_uses_gemm(const void* w, int kind, const float* y, int M, int K, int N) {
    const bool known = (kind >= 0 && kind <= 3) || kind == KIND_F16;
    return known && M >= GEMM_MIN_ROWS && K > 0 && K % 32 == 0 && (kind == KIND_F16 || K % 256 == 0) &&
           (reinterpret_cast<uintptr_t>(w) & 15) == 0 && N % 4 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0;
}

int linear_a16(const void* a16, const void* w, int kind, float* y, int M, int K, int N) {
    B200_REQUIRE(a16 && w && y && linear_uses_gemm(w, kind, y, M, K, N) && (reinterpret_cast<uintptr_t>(a16) & 15) == 0,
                 "linear_a16: shape outside the tensor-core path");
    const __half* a = static_cast<const __half*>(a16);
    if (kind == KIND_F16)
        return umma_gemm(GEMM_EPI_STORE, a, M, static_cast<const __half*>(w), nullptr, N, nullptr, 1, M, N, K, y, nullptr, N, 1.0f);
    return umma_gemm_q(GEMM_EPI_STORE, kind, a, M, w, nullptr, N, nullptr, 1, M, N, K, y, nullptr, N, 1.0f);
}

int linear(const float* x, const void* w, int kind, float* y, int M, int K, int N) {
    if (M <= 0 || N <= 0) return B200_OK;   // the reference returns silently too
    B200_REQUIRE(x && w && y, "linear: null pointer");
    B200_REQUIRE(K > 0, "linear: K must be positive");
    if (kind >= 0 && kind <= 3) {
        B200_REQUIRE(K % q_block_elems(kind) == 0, "linear_forward_q4: K must be a multiple of %d",
                     q_block_elems(kind));
    } else {
        B200_REQUIRE(kind == KIND_F32 || kind == KIND_F16, "linear: unknown weight kind %d", kind);
    }
    if (K % 32 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0 ||
        (kind == KIND_F16 && (reinterpret_cast<uintptr_t>(w) & 15) != 0) ||
        (kind == KIND_F32 && (reinterpret_cast<uintptr_t>(w) & 15) != 0)) {
        B200_REQUIRE(kind == KIND_F32 || kind == KIND_F16,
                     "linear_forward_q4: x must be 16-byte aligned");
        GemvArgs a{x, reinterpret_cast<const uint8_t*>(w), y, M, K, N};
        if (kind == KIND_F32) gemv_ragged_kernel<KIND_F32><<<ceil_div(N, 4), 128, 0, stream()>>>(a);
        else gemv_ragged_kernel<KIND_F16><<<ceil_div(N, 4), 128, 0, stream()>>>(a);
        B200_LAUNCH_CHECK("gemv_ragged_kernel");
        return B200_OK;
    }
    // Many tokens over fp16 or packed weights: tensor-core GEMM on fp16 copies of the
    // activations and (for packed kinds) of the weights.  fp32 weights stay on the
    // exact fp32 path.
    if (M >= GEMM_MIN_ROWS && kind != KIND_F32 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && N % 4 == 0 &&
        (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
        const size_t a_bytes = ((size_t)M * K * 2 + 255) & ~(size_t)255;
        const bool in_kernel = kind != KIND_F16 && K % 256 == 0;     // packed weights dequantised by the GEMM itself
        const size_t b_bytes = (kind == KIND_F16 || in_kernel) ? 0 : (size_t)N * K * 2;
        void* ws;
        int rc = workspace(WS_LINEAR).ensure(a_bytes + b_bytes + 256, &ws);
        if (rc) return rc;
        const __half* a16 = f16_shadow_find(x, M, K);       // rows a fused norm has already written as fp16
        if (!a16) {
            __half* packed = static_cast<__half*>(ws);
            rc = pack_rows_f16(x, nullptr, 1, packed, M, K);
            if (rc) return rc;
            a16 = packed;
        }
        if (in_kernel)
            return umma_gemm_q(GEMM_EPI_STORE, kind, a16, M, w, nullptr, N, nullptr, 1, M, N, K, y, nullptr, N, 1.0f);
        const __half* b16 = static_cast<const __half*>(w);
        if (kind != KIND_F16) {
            uint16_t* scratch = reinterpret_cast<uint16_t*>(static_cast<char*>(ws) + a_bytes);
            rc = dequantize(static_cast<const uint8_t*>(w), scratch, (int64_t)N * K, kind);
            if (rc) return rc;
            b16 = reinterpret_cast<const __half*>(scratch);
        }
        return umma_gemm(GEMM_EPI_STORE, a16, M, b16, nullptr, N, nullptr, 1, M, N, K, y, nullptr, N, 1.0f);
    }
    // Preferred path: the TMA-streamed kernel (tensor-core dot for Q4_K / fp16 weights),
    // eight tokens per pass.  Shapes it cannot tile fall through to the plain kernel.
    if ((reinterpret_cast<uintptr_t>(w) & 15) == 0 && (kind != 3 || K % 256 == 0)) {
        bool streamed = true;
        for (int m0 = 0; m0 < M && streamed; m0 += 8) {
            SgArgs s;
            s.w = reinterpret_cast<const uint8_t*>(w);
            s.N = N; s.K = K; s.M = std::min(8, M - m0);
            s.x = x + (int64_t)m0 * K; s.x_stride = K;
            s.y = y + (int64_t)m0 * N; s.y_stride = N;
            const int rc = stream_gemv(s, kind, PRO_NONE, EPI_STORE);
            if (rc == B200_EUNSUPPORTED && m0 == 0) streamed = false;
            else if (rc) return rc;
        }
        if (streamed) return B200_OK;
    }
    for (int m0 = 0; m0 < M; m0 += 8) {
        GemvArgs a{x + (int64_t)m0 * K, reinterpret_cast<const uint8_t*>(w), y + (int64_t)m0 * N,
                   std::min(8, M - m0), K, N};
        int rc;
        switch (kind) {
            case 0: rc = launch_gemv_kind<0>(a); break;
            case 1: rc = launch_gemv_kind<1>(a); break;
            case 2: rc = launch_gemv_kind<2>(a); break;
            case 3: rc = launch_gemv_kind<3>(a); break;
            case KIND_F16: rc = launch_gemv_kind<KIND_F16>(a); break;
            default: rc = launch_gemv_kind<KIND_F32>(a); break;
        }
        if (rc) return rc;
    }
    return B200_OK;
}

// ---------------------------------------------------------------------------
// split_qkv, converts (cuda/kernels.cu:104,451 and k_split_qkv)
// ---------------------------------------------------------------------------
__global__ void split_qkv_kernel(const float* __restrict__ qkv, float* __restrict__ q,
                                 float* __restrict__ k, float* __restrict__ v, int64_t n, int qd,
                                 int kvd) {
    const int w = qd + 2 * kvd;
    const int64_t total = n * w;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / w;
        const int c = (int)(i - r * w);
        const float val = qkv[i];
        if (c < qd) q[r * qd + c] = val;
        else if (c < qd + kvd) k[r * kvd + (c - qd)] = val;
        else v[r * kvd + (c - qd - kvd)] = val;
    }
}

__global__ void f32_to_f16_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = float_to_half_bits(src[i]);
}
__global__ void f16_to_f32_kernel(const uint16_t* __restrict__ src, float* __restrict__ dst, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = half_bits_to_float(src[i]);
}

static inline int flat_grid(int64_t n) {
    return (int)std::max<int64_t>(1, std::min<int64_t>(ceil_div64(n, 256), (int64_t)num_sms() * 16));
}

}  // namespace b200

using namespace b200;

// ---------------------------------------------------------------------------
// Self-test of the bounded wait every TMA-fed kernel of the library uses (mbar_wait):
// a barrier that expects one arrival and never gets it.  The wait gives up after
// `spin_limit` tries, raises the status word and the kernel returns normally.
// ---------------------------------------------------------------------------
namespace b200 {
__global__ void bounded_wait_probe_kernel(int* status, uint32_t limit, int* outcome) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) *outcome = mbar_wait_limit(&bar, 0, status, limit) ? 1 : 2;
}
}  // namespace b200

extern "C" int b200_test_bounded_wait(int spin_limit, int* outcome_dev) {
    B200_REQUIRE(spin_limit >= 1 && spin_limit <= (1 << 20) && outcome_dev, "test_bounded_wait: bad arguments");
    int* status = stream_status_ptr();
    B200_REQUIRE(status, "test_bounded_wait: no status word");
    bounded_wait_probe_kernel<<<1, 32, 0, stream()>>>(status, (uint32_t)spin_limit, outcome_dev);
    B200_LAUNCH_CHECK("bounded_wait_probe_kernel");
    return B200_OK;
}

extern "C" {

int b200_linear_forward(const float* x, const float* w, float* y, int M, int K, int N) {
    return linear(x, w, KIND_F32, y, M, K, N);
}
int b200_linear_forward_f32(const float* x, const float* w, float* y, int M, int K, int N) {
    return linear(x, w, KIND_F32, y, M, K, N);
}
int b200_linear_forward_fp16(const float* x, const uint16_t* w, float* y, int M, int K, int N) {
    return linear(x, w, KIND_F16, y, M, K, N);
}
int b200_linear_forward_q4(const float* x, const uint16_t* w, float* y, int M, int K, int N, int kind) {
    if (M <= 0 || N <= 0) return B200_OK;
    B200_REQUIRE(kind >= 0 && kind <= 3, "linear_forward_q4: unknown kind %d", kind);
    return linear(x, w, kind, y, M, K, N);
}
int b200_gemm(int trans_a, int trans_b, int M, int N, int K, float alpha, const float* A, int lda,
              const float* B, int ldb, float beta, float* C, int ldc) {
    if (M <= 0 || N <= 0) return B200_OK;
    if (trans_a || !trans_b || alpha != 1.0f || beta != 0.0f || lda != K || ldb != K || ldc != N)
        return fail(B200_EUNSUPPORTED,
                    "gemm: only C = A . B^T (alpha 1, beta 0, packed leading dimensions) is provided "
                    "by the inference backend");
    return linear(A, B, KIND_F32, C, M, K, N);
}
int b200_dequantize_quant(const uint16_t* src, uint16_t* dst, int64_t n, int kind) {
    return dequantize(reinterpret_cast<const uint8_t*>(src), dst, n, kind);
}

// 16 reusable fp16 scratch slots for materialised weights (cuda/kernels.cu:516-541).
static void* g_qslot[16];
static size_t g_qslot_bytes[16];
int b200_quant_scratch(int slot, int64_t n, uint16_t** out) {
    B200_REQUIRE(out && n > 0, "quant_scratch: bad arguments");
    if (slot < 0 || slot >= 16) slot = 0;
    const size_t need = (size_t)n * 2;
    if (g_qslot_bytes[slot] < need) {
        if (g_qslot[slot]) B200_CUDA(cudaFree(g_qslot[slot]));
        g_qslot[slot] = nullptr;
        g_qslot_bytes[slot] = 0;
        const size_t rounded = (need + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
        B200_CUDA(cudaMalloc(&g_qslot[slot], rounded));
        g_qslot_bytes[slot] = rounded;
    }
    *out = static_cast<uint16_t*>(g_qslot[slot]);
    return B200_OK;
}
int b200_free_quant_scratch(void) {
    for (int i = 0; i < 16; ++i) {
        if (g_qslot[i]) cudaFree(g_qslot[i]);
        g_qslot[i] = nullptr;
        g_qslot_bytes[i] = 0;
    }
    return B200_OK;
}

int b200_split_qkv(const float* qkv, float* q, float* k, float* v, int64_t n, int qd, int kvd) {
    if (n <= 0) return B200_OK;
    B200_REQUIRE(qkv && q && k && v && qd > 0 && kvd > 0, "split_qkv: bad arguments");
    split_qkv_kernel<<<flat_grid(n * (qd + 2 * kvd)), 256, 0, stream()>>>(qkv, q, k, v, n, qd, kvd);
    B200_LAUNCH_CHECK("split_qkv_kernel");
    return B200_OK;
}
int b200_convert_f32_to_f16(const float* src, uint16_t* dst, int64_t n) {
    if (n <= 0) return B200_OK;
    B200_REQUIRE(src && dst, "convert_f32_to_f16: null pointer");
    f32_to_f16_kernel<<<flat_grid(n), 256, 0, stream()>>>(src, dst, n);
    B200_LAUNCH_CHECK("f32_to_f16_kernel");
    return B200_OK;
}
int b200_convert_f16_to_f32(const uint16_t* src, float* dst, int64_t n) {
    if (n <= 0) return B200_OK;
    B200_REQUIRE(src && dst, "convert_f16_to_f32: null pointer");
    f16_to_f32_kernel<<<flat_grid(n), 256, 0, stream()>>>(src, dst, n);
    B200_LAUNCH_CHECK("f16_to_f32_kernel");
    return B200_OK;
}

}  // extern "C"
