// MoE layer for many tokens: expert-grouped tensor-core GEMMs.
//
// The token-major kernels of moe.cu read an expert's matrices once per (token, k)
// slot, which is right for a handful of tokens and hopeless for a prompt.  Here the
// slots are sorted by expert (the canonical stable permutation), their activations
// gathered into expert-contiguous fp16 rows, and each expert's gate/up and down
// projections run as one group of a grouped GEMM on tcgen05 (gemm_umma.cu):
//
//   route -> permutation -> gather rows (fp16) -> [gate|up] GEMM with SwiGLU epilogue
//         -> down GEMM -> combine: out[t] = shared(x_t) + sum_k w[t,k] * y[pos(t,k)]
//
// The combine adds the K expert outputs of a token in k order (no atomics), so the
// result is run-to-run bit-stable.  Reference: cpu::moe_forward_bias
// (core/moe_cpu.cpp:198-288); the reference's CUDA layer (cuda/moe.cu:731-958) makes
// 3 cuBLAS calls per expert and synchronises with the host for the group offsets.
#include "gemm.cuh"
#include "linear.cuh"

namespace b200 {

int moe_route(const float* x, const float* router_w, const float* router_bias, float* probs, int32_t* idx, float* w,
              int64_t N, int d, int ne, int K);
int moe_permutation(const int32_t* idx, int64_t NK, int ne, int32_t* grouped, int32_t* offsets);
int moe_permutation_inv(const int32_t* idx, int64_t NK, int ne, int32_t* grouped, int32_t* inv, int32_t* offsets);
int moe_permutation_small_max();

constexpr int GROUPED_CHUNK_TOKENS = 8192;

// inv[grouped[pos]] = pos
__global__ void perm_inverse_kernel(const int32_t* __restrict__ grouped, int32_t* __restrict__ inv, int64_t NK) {
    const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (p < NK) inv[grouped[p]] = (int32_t)p;
}

// out[t, :] = (shared ? out[t, :] : 0) + sum_k w[t,k] * y[inv[t*K + k], :]   (k ascending)
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ y, const int32_t* __restrict__ inv,
                                                         const float* __restrict__ w, float* __restrict__ out, int N,
                                                         int K, int d, int has_shared) {
    const int d4 = d >> 2;
    const int64_t total = (int64_t)N * d4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / d4), j = (int)(i - (int64_t)t * d4);
        float4* o = reinterpret_cast<float4*>(out + (int64_t)t * d) + j;
        float4 acc = has_shared ? *o : make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < K; ++k) {
            const int slot = t * K + k;
            const float wk = w[slot];
            const float4 v = *(reinterpret_cast<const float4*>(y + (int64_t)inv[slot] * d) + j);
            acc.x = __fadd_rn(acc.x, __fmul_rn(wk, v.x));
            acc.y = __fadd_rn(acc.y, __fmul_rn(wk, v.y));
            acc.z = __fadd_rn(acc.z, __fmul_rn(wk, v.z));
            acc.w = __fadd_rn(acc.w, __fmul_rn(wk, v.w));
        }
        *o = acc;
    }
}

// kind: template tag (KIND_F16 or a packed kind).  Pointers as in moe_forward().
int moe_forward_grouped(const float* x, const float* router_w, const float* router_bias, const void* gates,
                        const void* ups, const void* downs, const void* sh_g, const void* sh_u, const void* sh_d,
                        float* out, float* probs_cache, int32_t* idx_cache, float* w_cache, int64_t N, int d, int E,
                        int ne, int K, int SH, int kind) {
    const bool shared = sh_g && sh_u && sh_d && SH > 0;
    const int64_t chunk = std::min<int64_t>(N, GROUPED_CHUNK_TOKENS);
    const size_t CK = (size_t)chunk * K;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off += (bytes + 255) & ~(size_t)255; return o; };
    const size_t we = (size_t)ne * E * d, ws = (size_t)SH * d;
    // packed experts are dequantised inside the GEMM when every contraction length is a
    // multiple of 256; otherwise through fp16 copies made once per call
    const bool in_kernel = kind != KIND_F16 && d % 256 == 0 && E % 256 == 0 && (!shared || SH % 256 == 0);
    const bool packed = kind != KIND_F16 && !in_kernel;
    const size_t o_g = packed ? take(we * 2) : 0, o_u = packed ? take(we * 2) : 0, o_d = packed ? take(we * 2) : 0;
    const size_t o_sg = packed && shared ? take(ws * 2) : 0, o_su = packed && shared ? take(ws * 2) : 0,
                 o_sd = packed && shared ? take(ws * 2) : 0;
    const size_t o_idx = take(CK * 4), o_w = take(CK * 4), o_grp = take(CK * 4), o_inv = take(CK * 4),
                 o_off = take((size_t)(ne + 1) * 4);
    const size_t o_a = take(CK * d * 2), o_act = take(CK * E * 2), o_y = take(CK * d * 4);
    const size_t o_xs = shared ? take((size_t)chunk * d * 2) : 0, o_sact = shared ? take((size_t)chunk * SH * 2) : 0;
    void* wsp;
    int rc = workspace(WS_MOE).ensure(off + 256, &wsp);
    if (rc) return rc;
    char* base = static_cast<char*>(wsp);
    auto H = [&](size_t o) { return reinterpret_cast<__half*>(base + o); };

    // fp16 copies of packed weights, once per call
    const __half *g16 = static_cast<const __half*>(gates), *u16 = static_cast<const __half*>(ups),
                 *d16 = static_cast<const __half*>(downs), *sg16 = static_cast<const __half*>(sh_g),
                 *su16 = static_cast<const __half*>(sh_u), *sd16 = static_cast<const __half*>(sh_d);
    if (packed) {
        auto deq = [&](const void* src, size_t o, size_t n) {
            return dequantize(static_cast<const uint8_t*>(src), reinterpret_cast<uint16_t*>(base + o), (int64_t)n, kind);
        };
        if ((rc = deq(gates, o_g, we)) || (rc = deq(ups, o_u, we)) || (rc = deq(downs, o_d, we))) return rc;
        g16 = H(o_g); u16 = H(o_u); d16 = H(o_d);
        if (shared) {
            if ((rc = deq(sh_g, o_sg, ws)) || (rc = deq(sh_u, o_su, ws)) || (rc = deq(sh_d, o_sd, ws))) return rc;
            sg16 = H(o_sg); su16 = H(o_su); sd16 = H(o_sd);
        }
    }

    auto gemm = [&](int epi, const __half* A, int64_t a_rows, const void* Bq, const void* Bq2, const __half* B16,
                    const __half* B16b, int64_t b_rows, const int32_t* offs, int groups, int M, int Nn, int Kk, float* c,
                    __half* c16, int64_t ldc, bool split_k_ok = true) {
        if (in_kernel)
            return umma_gemm_q(epi, kind, A, a_rows, Bq, Bq2, b_rows, offs, groups, M, Nn, Kk, c, c16, ldc, 1.0f, nullptr,
                               nullptr, split_k_ok);
        return umma_gemm(epi, A, a_rows, B16, B16b, b_rows, offs, groups, M, Nn, Kk, c, c16, ldc, 1.0f);
    };

    for (int64_t t0 = 0; t0 < N; t0 += chunk) {
        const int T = (int)std::min<int64_t>(chunk, N - t0);
        const int64_t NK = (int64_t)T * K;
        const float* xc = x + t0 * d;
        float* oc = out + t0 * d;
        int32_t* idx = idx_cache ? idx_cache + t0 * K : reinterpret_cast<int32_t*>(base + o_idx);
        float* w = w_cache ? w_cache + t0 * K : reinterpret_cast<float*>(base + o_w);
        int32_t* grouped = reinterpret_cast<int32_t*>(base + o_grp);
        int32_t* inv = reinterpret_cast<int32_t*>(base + o_inv);
        int32_t* offsets = reinterpret_cast<int32_t*>(base + o_off);
        float* y = reinterpret_cast<float*>(base + o_y);

        // The shared expert shares no data with routing, permutation, gather and the routed
        // experts until the combine: it runs on the side stream next to them, straight into out.
        if (shared) {
            if ((rc = side_begin())) return rc;
            rc = pack_rows_f16(xc, nullptr, 1, H(o_xs), T, d);
            if (!rc)
                rc = gemm(GEMM_EPI_SWIGLU, H(o_xs), T, sh_g, sh_u, sg16, su16, SH, nullptr, 1, T, SH, d, nullptr,
                          H(o_sact), SH);
            if (!rc)
                // (one K range always: the expert-parallel layer runs the same product on a slice of
                // the tokens and must reproduce these bits)
                rc = gemm(GEMM_EPI_STORE, H(o_sact), T, sh_d, nullptr, sd16, nullptr, d, nullptr, 1, T, d, SH, oc, nullptr, d,
                          false);
            const int rc2 = side_end();
            if (rc) return rc;
            if (rc2) return rc2;
        }
        rc = moe_route(xc, router_w, router_bias, probs_cache ? probs_cache + t0 * ne : nullptr, idx, w, T, d, ne, K);
        if (rc) return rc;
        rc = moe_permutation(idx, NK, ne, grouped, offsets);
        if (rc) return rc;
        perm_inverse_kernel<<<(unsigned)ceil_div64(NK, 256), 256, 0, stream()>>>(grouped, inv, NK);
        B200_LAUNCH_CHECK("perm_inverse_kernel");
        rc = pack_rows_f16(xc, grouped, K, H(o_a), NK, d);
        if (rc) return rc;
        // routed experts
        rc = gemm(GEMM_EPI_SWIGLU, H(o_a), NK, gates, ups, g16, u16, (int64_t)ne * E, offsets, ne, (int)NK, E, d, nullptr,
                  H(o_act), E);
        if (rc) return rc;
        rc = gemm(GEMM_EPI_STORE, H(o_act), NK, downs, nullptr, d16, nullptr, (int64_t)ne * d, offsets, ne, (int)NK, d, E,
                  y, nullptr, d);
        if (rc) return rc;
        if (shared && (rc = side_wait())) return rc;
        const int64_t total = (int64_t)T * (d >> 2);
        const int grid = (int)std::min<int64_t>(ceil_div64(total, 256), (int64_t)num_sms() * 16);
        moe_combine_kernel<<<grid, 256, 0, stream()>>>(y, inv, w, oc, T, K, d, shared ? 1 : 0);
        B200_LAUNCH_CHECK("moe_combine_kernel");
    }
    return B200_OK;
}

// ===========================================================================
// A decode batch (more tokens than the token-major kernels take, fewer than fill the
// tensor-core tiles of every expert): routing and permutation as above, the routed experts
// through moe_units.cu, the shared expert as a GEMM on the side stream, the same k-ordered
// combination.
// ===========================================================================
int moe_combine(const float* y, const int32_t* inv, const float* w, float* out, int64_t N, int d, int K, bool accumulate);
int moe_forward_units(const float* x, const float* router_w, const float* router_bias, const void* gates,
                      const void* ups, const void* downs, const void* sh_g, const void* sh_u, const void* sh_d,
                      float* out, float* probs_cache, int32_t* idx_cache, float* w_cache, int64_t N, int d, int E,
                      int ne, int K, int SH, int kind) {
    const bool shared = sh_g && sh_u && sh_d && SH > 0;
    const size_t NK = (size_t)N * K;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off += (bytes + 255) & ~(size_t)255; return o; };
    const size_t o_idx = take(NK * 4), o_w = take(NK * 4), o_grp = take(NK * 4), o_inv = take(NK * 4),
                 o_off = take((size_t)(ne + 1) * 4), o_units = take(moe_units_table_bytes((int64_t)NK, ne)),
                 o_act = take(NK * E * 4), o_y = take(NK * d * 4),
                 o_sh = shared ? take(moe_shared_scratch_bytes(N, d, SH)) : 0;
    void* wsp;
    int rc = workspace(WS_MOE).ensure(off + 256, &wsp);
    if (rc) return rc;
    char* base = static_cast<char*>(wsp);
    int32_t* idx = idx_cache ? idx_cache : reinterpret_cast<int32_t*>(base + o_idx);
    float* w = w_cache ? w_cache : reinterpret_cast<float*>(base + o_w);
    int32_t* grouped = reinterpret_cast<int32_t*>(base + o_grp);
    int32_t* inv = reinterpret_cast<int32_t*>(base + o_inv);
    int32_t* offsets = reinterpret_cast<int32_t*>(base + o_off);
    float* act = reinterpret_cast<float*>(base + o_act);
    float* y = reinterpret_cast<float*>(base + o_y);
    if (shared) {
        if ((rc = side_begin())) return rc;
        rc = moe_shared_expert(x, sh_g, sh_u, sh_d, out, N, d, SH, kind, base + o_sh);
        const int rc2 = side_end();
        if (rc) return rc;
        if (rc2) return rc2;
    }
    rc = moe_route(x, router_w, router_bias, probs_cache, idx, w, N, d, ne, K);
    if (rc) return rc;
    rc = moe_dispatch_perm(idx, N, ne, K, grouped, inv, offsets);
    if (rc) return rc;
    rc = moe_units_forward(x, grouped, offsets, gates, ups, downs, act, y, base + o_units, N, d, E, ne, K, kind);
    if (rc) return rc;
    if (shared && (rc = side_wait())) return rc;
    return moe_combine(y, inv, w, out, N, d, K, shared);
}

// ===========================================================================
// The same layer cut at its exchange points, for expert parallelism: a rank routes
// and packs its own tokens (rows come out sorted by expert, hence by owning rank),
// the rows travel, the owner runs its experts on whatever rows arrived - one group
// per (source rank, local expert) block, in arrival order - the results travel back
// and the token's owner combines them.  Each function is stream-ordered and keeps
// no state between calls.
// ===========================================================================
static int check_ep_kind(const char* who, int kind, int d, int E) {
    B200_REQUIRE(kind == KIND_F16 || (kind >= 0 && kind <= 3), "%s: experts must be fp16 or packed", who);
    B200_REQUIRE(d % 32 == 0 && E % 32 == 0, "%s: d and E must be multiples of 32", who);
    if (kind != KIND_F16 && (d % 256 != 0 || E % 256 != 0))
        return fail(B200_EUNSUPPORTED, "%s: packed experts need d and E to be multiples of 256", who);
    return B200_OK;
}

// The permutation alone: grouped [N K] (slot numbers sorted by expert, stable), its inverse
// and the expert offsets [ne + 1].
int moe_dispatch_perm(const int32_t* idx, int64_t N, int ne, int K, int32_t* grouped, int32_t* inv, int32_t* offsets) {
    B200_REQUIRE(idx && grouped && inv && offsets, "moe_dispatch_perm: null pointer");
    const int64_t NK = N * K;
    if (NK <= 0) return B200_OK;
    if (NK <= moe_permutation_small_max()) return moe_permutation_inv(idx, NK, ne, grouped, inv, offsets);
    const int rc = moe_permutation(idx, NK, ne, grouped, offsets);
    if (rc) return rc;
    perm_inverse_kernel<<<(unsigned)ceil_div64(NK, 256), 256, 0, stream()>>>(grouped, inv, NK);
    B200_LAUNCH_CHECK("perm_inverse_kernel");
    return B200_OK;
}

int moe_dispatch_pack(const float* x, const int32_t* idx, int64_t N, int d, int ne, int K, __half* rows16, int32_t* inv,
                      int32_t* offsets) {
    B200_REQUIRE(x && idx && rows16 && inv && offsets, "moe_dispatch_pack: null pointer");
    const int64_t NK = N * K;
    if (NK <= 0) return B200_OK;
    void* wsp;
    int rc = workspace(WS_MOE).ensure((size_t)NK * 4 + 256, &wsp);
    if (rc) return rc;
    int32_t* grouped = static_cast<int32_t*>(wsp);
    rc = moe_permutation(idx, NK, ne, grouped, offsets);
    if (rc) return rc;
    perm_inverse_kernel<<<(unsigned)ceil_div64(NK, 256), 256, 0, stream()>>>(grouped, inv, NK);
    B200_LAUNCH_CHECK("perm_inverse_kernel");
    return pack_rows_f16(x, grouped, K, rows16, NK, d);
}

int moe_experts_rows(const __half* rows16, const int32_t* offsets, const int32_t* group_map, int groups, int64_t R,
                     const void* gates, const void* ups, const void* downs, int n_local, float* y, int d, int E,
                     int kind, float* const* y_groups) {
    if (R <= 0) return B200_OK;
    B200_REQUIRE(rows16 && offsets && gates && ups && downs && (y || y_groups) && groups >= 1 && n_local >= 1,
                 "moe_experts_rows: bad arguments");
    int rc = check_ep_kind("moe_experts_rows", kind, d, E);
    if (rc) return rc;
    void* wsp;
    rc = workspace(WS_MOE).ensure((size_t)R * E * 2 + 256, &wsp);
    if (rc) return rc;
    __half* act = static_cast<__half*>(wsp);
    if (kind == KIND_F16) {
        rc = umma_gemm(GEMM_EPI_SWIGLU, rows16, R, static_cast<const __half*>(gates), static_cast<const __half*>(ups),
                       (int64_t)n_local * E, offsets, groups, (int)R, E, d, nullptr, act, E, 1.0f, group_map);
        if (rc) return rc;
        return umma_gemm(GEMM_EPI_STORE, act, R, static_cast<const __half*>(downs), nullptr, (int64_t)n_local * d, offsets,
                         groups, (int)R, d, E, y, nullptr, d, 1.0f, group_map, y_groups);
    }
    rc = umma_gemm_q(GEMM_EPI_SWIGLU, kind, rows16, R, gates, ups, (int64_t)n_local * E, offsets, groups, (int)R, E, d,
                     nullptr, act, E, 1.0f, group_map);
    if (rc) return rc;
    return umma_gemm_q(GEMM_EPI_STORE, kind, act, R, downs, nullptr, (int64_t)n_local * d, offsets, groups, (int)R, d, E, y,
                       nullptr, d, 1.0f, group_map, y_groups);
}

// out [N, d] = shared_expert(x); false "shared" (a null matrix or SH == 0) leaves out untouched.
// scratch (optional): moe_shared_scratch_bytes(N, d, SH) bytes of the caller's instead of the
// library's MoE workspace (callers that run this next to the routed experts' GEMMs).
size_t moe_shared_scratch_bytes(int64_t N, int d, int SH) {
    return (((size_t)N * d * 2 + 255) & ~(size_t)255) + (size_t)N * SH * 2 + 256;
}
int moe_shared_expert(const float* x, const void* sh_g, const void* sh_u, const void* sh_d, float* out, int64_t N, int d,
                      int SH, int kind, void* scratch) {
    if (N <= 0) return B200_OK;
    if (!(sh_g && sh_u && sh_d && SH > 0)) return B200_OK;
    B200_REQUIRE(x && out, "moe_shared_expert: null pointer");
    int rc = check_ep_kind("moe_shared_combine", kind, d, SH);
    if (rc) return rc;
    void* wsp = scratch;
    const size_t xs_bytes = ((size_t)N * d * 2 + 255) & ~(size_t)255;
    if (!wsp) {
        rc = workspace(WS_MOE).ensure(moe_shared_scratch_bytes(N, d, SH), &wsp);
        if (rc) return rc;
    }
    const __half* xs = f16_shadow_find(x, N, d);           // rows a fused norm has already written as fp16
    __half* sact = reinterpret_cast<__half*>(static_cast<char*>(wsp) + xs_bytes);
    if (!xs) {
        __half* packed = static_cast<__half*>(wsp);
        rc = pack_rows_f16(x, nullptr, 1, packed, N, d);
        if (rc) return rc;
        xs = packed;
    }
    if (kind == KIND_F16) {
        rc = umma_gemm(GEMM_EPI_SWIGLU, xs, N, static_cast<const __half*>(sh_g), static_cast<const __half*>(sh_u), SH,
                       nullptr, 1, (int)N, SH, d, nullptr, sact, SH, 1.0f);
        if (rc) return rc;
        return umma_gemm(GEMM_EPI_STORE, sact, N, static_cast<const __half*>(sh_d), nullptr, d, nullptr, 1, (int)N, d, SH,
                         out, nullptr, d, 1.0f);
    }
    rc = umma_gemm_q(GEMM_EPI_SWIGLU, kind, xs, N, sh_g, sh_u, SH, nullptr, 1, (int)N, SH, d, nullptr, sact, SH, 1.0f);
    if (rc) return rc;
    // one K range always: a token's result must not depend on how many tokens the call has
    // (the expert-parallel layer runs this on a slice and must reproduce the single GPU's bits)
    return umma_gemm_q(GEMM_EPI_STORE, kind, sact, N, sh_d, nullptr, d, nullptr, 1, (int)N, d, SH, out, nullptr, d, 1.0f,
                       nullptr, nullptr, false);
}

// out [N, d] (+)= sum_k w[t, k] * y[inv[t K + k]] in k order; accumulate: onto the shared
// expert's result already in out.
int moe_combine(const float* y, const int32_t* inv, const float* w, float* out, int64_t N, int d, int K, bool accumulate) {
    if (N <= 0) return B200_OK;
    B200_REQUIRE(y && inv && w && out && d % 4 == 0, "moe_combine: bad arguments");
    const int64_t total = N * (d >> 2);
    const int grid = (int)std::min<int64_t>(ceil_div64(total, 256), (int64_t)num_sms() * 16);
    moe_combine_kernel<<<grid, 256, 0, stream()>>>(y, inv, w, out, (int)N, K, d, accumulate ? 1 : 0);
    B200_LAUNCH_CHECK("moe_combine_kernel");
    return B200_OK;
}

int moe_shared_combine(const float* x, const void* sh_g, const void* sh_u, const void* sh_d, const float* y,
                       const int32_t* inv, const float* w, float* out, int64_t N, int d, int K, int SH, int kind) {
    if (N <= 0) return B200_OK;
    B200_REQUIRE(x && y && inv && w && out && d % 4 == 0, "moe_shared_combine: bad arguments");
    const bool shared = sh_g && sh_u && sh_d && SH > 0;
    const int rc = moe_shared_expert(x, sh_g, sh_u, sh_d, out, N, d, SH, kind, nullptr);
    if (rc) return rc;
    return moe_combine(y, inv, w, out, N, d, K, shared);
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_moe_route(const float* x, const float* router_w, const float* router_bias, float* probs, int32_t* idx,
                   float* w, int64_t N, int d, int ne, int K) {
    if (N <= 0) return B200_OK;
    B200_REQUIRE(x && router_w && idx && w, "moe_route: null pointer");
    B200_REQUIRE(K >= 1 && K <= 16 && ne >= K && ne <= 256 && d > 0 && d % 4 == 0, "moe_route: K / ne / d out of range");
    return moe_route(x, router_w, router_bias, probs, idx, w, N, d, ne, K);
}
int b200_moe_dispatch_pack(const float* x, const int32_t* idx, int64_t N, int d, int ne, int K, uint16_t* rows16,
                           int32_t* inv, int32_t* offsets) {
    return moe_dispatch_pack(x, idx, N, d, ne, K, reinterpret_cast<__half*>(rows16), inv, offsets);
}
int b200_moe_experts_rows(const uint16_t* rows16, const int32_t* offsets, const int32_t* group_map, int groups,
                          int64_t R, const void* gates, const void* ups, const void* downs, int n_local, float* y, int d,
                          int E, int qkind) {
    B200_REQUIRE(qkind >= -1 && qkind <= 3, "moe_experts_rows: unknown qkind %d", qkind);
    return moe_experts_rows(reinterpret_cast<const __half*>(rows16), offsets, group_map, groups, R, gates, ups, downs,
                            n_local, y, d, E, tag_of_qkind(qkind), nullptr);
}
int b200_moe_shared_expert(const float* x, const void* sh_g, const void* sh_u, const void* sh_d, float* out, int64_t N,
                           int d, int SH, int qkind) {
    B200_REQUIRE(qkind >= -1 && qkind <= 3, "moe_shared_expert: unknown qkind %d", qkind);
    return moe_shared_expert(x, sh_g, sh_u, sh_d, out, N, d, SH, tag_of_qkind(qkind), nullptr);
}
int b200_moe_combine(const float* y, const int32_t* inv, const float* w, float* out, int64_t N, int d, int K,
                     int accumulate) {
    return moe_combine(y, inv, w, out, N, d, K, accumulate != 0);
}
int b200_moe_shared_combine(const float* x, const void* sh_g, const void* sh_u, const void* sh_d, const float* y,
                            const int32_t* inv, const float* w, float* out, int64_t N, int d, int K, int SH, int qkind) {
    B200_REQUIRE(qkind >= -1 && qkind <= 3, "moe_shared_combine: unknown qkind %d", qkind);
    return moe_shared_combine(x, sh_g, sh_u, sh_d, y, inv, w, out, N, d, K, SH, tag_of_qkind(qkind));
}

}  // extern "C"
