// Host interface of the tensor-core GEMM (gemm_umma.cu).
#pragma once

#include <cuda_fp16.h>

#include "common.cuh"

namespace b200 {

enum { GEMM_EPI_STORE = 0, GEMM_EPI_SWIGLU = 1 };

// From this many activation rows on, linear layers over fp16 or packed weights run
// on the tensor cores (activations rounded to fp16, as the reference's cuBLAS path
// does); below it they stream the weights once through the GEMV kernels in fp32.
constexpr int GEMM_MIN_ROWS = 32;

// dst[r, :] = fp16(src[(row_map ? row_map[r] / div : r), :]); K % 8 == 0.
int pack_rows_f16(const float* src, const int32_t* row_map, int div, __half* dst, int64_t rows, int K);
// The fp16 copy a producer registered for exactly these rows (f16_shadow_set), or null; see gemm_umma.cu.
void f16_shadow_set(const float* src, const __half* rows16, int64_t rows, int K);
void f16_shadow_clear();
const __half* f16_shadow_find(const float* src, int64_t rows, int K);

// C = A . B^T on tcgen05.  A [a_rows, K] fp16, B (and B2) [b_rows, K] fp16, fp32
// accumulation.  Rows of A form `groups` consecutive ranges given by the device
// array offsets[groups + 1] (null: one group of all M rows); range g uses rows
// [g*N, (g+1)*N) of B - or block group_map[g] when that device array is given.
//   GEMM_EPI_STORE   c[row, n]   = scale * acc                      (fp32, ld = ldc)
//   GEMM_EPI_SWIGLU  c16[row, n] = silu(A.B^T) * (A.B2^T)           (fp16, ld = ldc)
int umma_gemm(int epi, const __half* A, int64_t a_rows, const __half* B, const __half* B2, int64_t b_rows,
              const int32_t* offsets, int groups, int M, int N, int K, float* c, __half* c16, int64_t ldc, float scale,
              const int32_t* group_map = nullptr, float* const* group_c = nullptr);

// The same with B (and B2) in packed form, `kind` 0..3, dequantised inside the kernel
// (values rounded to fp16).  K % 256 == 0.  allow_split_k = false: K is never cut across CTAs,
// so a row's result does not depend on how many rows the call has (callers that must give
// the same bits for any slice of the rows).
int umma_gemm_q(int epi, int kind, const __half* A, int64_t a_rows, const void* B, const void* B2, int64_t b_rows,
                const int32_t* offsets, int groups, int M, int N, int K, float* c, __half* c16, int64_t ldc,
                float scale, const int32_t* group_map = nullptr, float* const* group_c = nullptr,
                bool allow_split_k = true);

// moe_grouped.cu: the shared expert alone, out [N, d] = shared_expert(x); kind is a template
// tag; scratch (optional) replaces the library's MoE workspace.
// The routed experts on packed rows (see b200_moe_experts_rows).  y_groups (optional, device
// [groups]): where each group's result rows go instead of y, in umma_gemm's group_c
// convention; y may then be null.
int moe_experts_rows(const __half* rows16, const int32_t* offsets, const int32_t* group_map, int groups, int64_t R,
                     const void* gates, const void* ups, const void* downs, int n_local, float* y, int d, int E, int kind,
                     float* const* y_groups = nullptr);
// moe_units.cu: the routed experts of a decode batch as weight streams shared by the tokens
// that chose them (few-token dot engine, exact dequantised weights).
size_t moe_units_table_bytes(int64_t NK, int ne);
int moe_units_forward(const float* x, const int32_t* grouped, const int32_t* offsets, const void* gates, const void* ups,
                      const void* downs, float* act, float* y, void* units_scratch, int64_t N, int d, int E, int ne, int K,
                      int kind);
int moe_dispatch_perm(const int32_t* idx, int64_t N, int ne, int K, int32_t* grouped, int32_t* inv, int32_t* offsets);
size_t moe_shared_scratch_bytes(int64_t N, int d, int SH);
int moe_shared_expert(const float* x, const void* sh_g, const void* sh_u, const void* sh_d, float* out, int64_t N, int d,
                      int SH, int kind, void* scratch);

}  // namespace b200
