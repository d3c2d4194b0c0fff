// Mixture-of-experts layer: router (softmax + top-K), deterministic expert
// permutation, routed SwiGLU experts + shared expert, weighted combine.
//
// Reference arithmetic: cpu::moe_forward_bias, core/moe_cpu.cpp:198-288 (router
// dot order :76-83, softmax core/math_cpu.cpp:546-558, top-K :85-98); kernels
// replaced: cuda/moe.cu:170-333 (route), :623-651 (grouping), :731-958 (layer).
//
// Routing is reproduced bit for bit: the router logit of (token, expert) is the
// fp32 chain s += ((a0*b0 + a1*b1) + a2*b2) + a3*b3 over groups of four in k order
// with unfused multiplies and adds; the softmax sums in expert order; selection is
// strict '>' in ascending expert order (lowest index wins ties).  Expert outputs
// are combined per token in k order (no atomics), so results are run-to-run
// bit-stable.
#include "gemm.cuh"
#include "linear.cuh"
#include "route.cuh"

namespace b200 {

// moe_grouped.cu
constexpr int MOE_UNITS_MAX_ROWS = 12;
int moe_forward_units(const float* x, const float* router_w, const float* router_bias, const void* gates,
                      const void* ups, const void* downs, const void* sh_g, const void* sh_u, const void* sh_d,
                      float* out, float* probs_cache, int32_t* idx_cache, float* w_cache, int64_t N, int d, int E,
                      int ne, int K, int SH, int kind);
int moe_forward_grouped(const float* x, const float* router_w, const float* router_bias, const void* gates,
                        const void* ups, const void* downs, const void* sh_g, const void* sh_u, const void* sh_d,
                        float* out, float* probs_cache, int32_t* idx_cache, float* w_cache, int64_t N, int d, int E,
                        int ne, int K, int SH, int kind);

constexpr int MOE_MAX_NE = 256;
constexpr int MOE_MAX_K = 16;

// ---------------------------------------------------------------------------
// Router: one block per token.
//   phase A  all threads: group sums g[i][e] = ((a0b0+a1b1)+a2b2)+a3b3 -> smem
//   phase B  thread e: the serial chain over the groups (and the scalar tail)
//   then     softmax in expert order, K rounds of warp arg-max, renormalise
// Shared memory: x[d] + g[chunk_groups][ne + 1] floats.
// ---------------------------------------------------------------------------
constexpr int ROUTE_THREADS = 256;

__global__ void __launch_bounds__(ROUTE_THREADS)
moe_route_kernel(const float* __restrict__ x, const float* __restrict__ router_w,
                 const float* __restrict__ router_bias, float* __restrict__ probs_out,
                 int32_t* __restrict__ idx_out, float* __restrict__ w_out, int d, int ne, int K,
                 int chunk_groups) {
    extern __shared__ float sm[];
    float* sx = sm;                          // [d]
    float* sg = sm + ((d + 3) & ~3);         // [chunk_groups][ne + 1] (padded: conflict-free both ways)
    __shared__ float s_logit[MOE_MAX_NE];    // logits -> exp -> probs
    __shared__ float s_sel[MOE_MAX_NE];
    __shared__ int s_idx[MOE_MAX_K];
    __shared__ float s_inv;
    const int64_t t = blockIdx.x;
    const float* xt = x + t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) sx[i] = xt[i];
    const int groups = d >> 2;
    float chain = 0.0f;                      // thread e's running sum
    for (int g0 = 0; g0 < groups; g0 += chunk_groups) {
        const int ng = min(chunk_groups, groups - g0);
        __syncthreads();
        // phase A: item = (e, gi) with gi fastest so a thread's loads walk a weight row
        for (int item = threadIdx.x; item < ng * ne; item += blockDim.x) {
            const int e = item / ng, gi = item - e * ng;
            const int k = (g0 + gi) << 2;
            const float4 b = *reinterpret_cast<const float4*>(router_w + (int64_t)e * d + k);
            const float4 a = *reinterpret_cast<const float4*>(sx + k);
            float g = __fadd_rn(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y));
            g = __fadd_rn(g, __fmul_rn(a.z, b.z));
            g = __fadd_rn(g, __fmul_rn(a.w, b.w));
            sg[gi * (ne + 1) + e] = g;
        }
        __syncthreads();
        // phase B
        if (threadIdx.x < ne) {
            const int e = threadIdx.x;
#pragma unroll 8
            for (int gi = 0; gi < ng; ++gi) chain = __fadd_rn(chain, sg[gi * (ne + 1) + e]);
        }
    }
    if (threadIdx.x < ne) {
        const int e = threadIdx.x;
        for (int k = groups << 2; k < d; ++k)
            chain = __fadd_rn(chain, __fmul_rn(sx[k], router_w[(int64_t)e * d + k]));
        s_logit[e] = chain;
    }
    __syncthreads();
    // softmax: max (order-free), exp, then the sum in expert order by one thread
    if (threadIdx.x < 32) {
        float mx = s_logit[0];
        for (int e = threadIdx.x; e < ne; e += 32) mx = fmaxf(mx, s_logit[e]);
        mx = warp_max(mx);
        // exp in double, rounded to float: matches the CPU libm's correctly rounded expf
        for (int e = threadIdx.x; e < ne; e += 32)
            s_logit[e] = (float)exp((double)__fsub_rn(s_logit[e], mx));
        __syncwarp();
        if (threadIdx.x == 0) {
            float sum = 0.0f;
            for (int e = 0; e < ne; ++e) sum = __fadd_rn(sum, s_logit[e]);
            s_inv = (sum > 1e-12f) ? __fdiv_rn(1.0f, sum) : 0.0f;
        }
        __syncwarp();
        const float inv = s_inv;
        for (int e = threadIdx.x; e < ne; e += 32) {
            const float p = __fmul_rn(s_logit[e], inv);
            s_logit[e] = p;
            s_sel[e] = router_bias ? __fadd_rn(p, router_bias[e]) : p;
        }
        __syncwarp();
        // K rounds of arg-max: value descending, index ascending; candidates must
        // exceed -1e30 (the reference's initial best value); none left -> expert 0.
        for (int k = 0; k < K; ++k) {
            float bv = -1e30f;
            int bi = -1;
            for (int e = threadIdx.x; e < ne; e += 32) {
                bool taken = false;
                for (int j = 0; j < k; ++j) taken |= (s_idx[j] == e);
                const float v = s_sel[e];
                if (!taken && v > bv) { bv = v; bi = e; }   // ascending e: strict '>' keeps the lowest
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
            }
            if (threadIdx.x == 0) s_idx[k] = bi < 0 ? 0 : bi;
            __syncwarp();
        }
        if (threadIdx.x == 0) {
            float tw[MOE_MAX_K];
            float sum_w = 0.0f;
            for (int k = 0; k < K; ++k) { tw[k] = s_logit[s_idx[k]]; sum_w = __fadd_rn(sum_w, tw[k]); }
            if (sum_w > 1e-8f) {
                const float inv_w = __fdiv_rn(1.0f, sum_w);
                for (int k = 0; k < K; ++k) tw[k] = __fmul_rn(tw[k], inv_w);
            } else {
                const float uni = __fdiv_rn(1.0f, (float)K);
                for (int k = 0; k < K; ++k) tw[k] = uni;
            }
            for (int k = 0; k < K; ++k) {
                idx_out[t * K + k] = s_idx[k];
                w_out[t * K + k] = tw[k];
            }
        }
        if (probs_out)
            for (int e = threadIdx.x; e < ne; e += 32) probs_out[t * ne + e] = s_logit[e];
    }
}

// ---------------------------------------------------------------------------
// Expert permutation: stable counting sort of slots s = t*K + k by expert.
// Three kernels, no atomics on ordering: per-block histograms, a scan over
// (expert, block), then a fill where each warp ranks its 32 slots with
// __match_any_sync and warps are ordered through shared-memory prefix sums.
// ---------------------------------------------------------------------------
constexpr int PERM_THREADS = 256;
constexpr int PERM_ITERS = 4;                              // slots per block = 256 * 4
constexpr int PERM_CHUNK = PERM_THREADS * PERM_ITERS;

__global__ void __launch_bounds__(PERM_THREADS)
perm_count_kernel(const int32_t* __restrict__ idx, int64_t NK, int ne, int32_t* __restrict__ block_counts) {
    __shared__ int cnt[MOE_MAX_NE];
    for (int e = threadIdx.x; e < ne; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    const int64_t base = (int64_t)blockIdx.x * PERM_CHUNK;
    for (int it = 0; it < PERM_ITERS; ++it) {
        const int64_t s = base + it * PERM_THREADS + threadIdx.x;
        if (s < NK) atomicAdd(&cnt[idx[s]], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < ne; e += blockDim.x) block_counts[(int64_t)blockIdx.x * ne + e] = cnt[e];
}

// One block; thread e walks the blocks of expert e.  block_counts becomes the
// first output position of (block, expert); offsets[ne+1] the expert boundaries.
__global__ void perm_scan_kernel(int32_t* __restrict__ block_counts, int nblocks, int ne,
                                 int32_t* __restrict__ offsets) {
    __shared__ int total[MOE_MAX_NE + 1];
    const int e = threadIdx.x;
    if (e < ne) {
        int run = 0;
        for (int b = 0; b < nblocks; ++b) {
            const int c = block_counts[(int64_t)b * ne + e];
            block_counts[(int64_t)b * ne + e] = run;
            run += c;
        }
        total[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < ne; ++i) { const int c = total[i]; total[i] = run; run += c; }
        total[ne] = run;
    }
    __syncthreads();
    if (e <= ne) offsets[e] = total[e];
    if (e < ne) {
        const int off = total[e];
        for (int b = 0; b < nblocks; ++b) block_counts[(int64_t)b * ne + e] += off;
    }
}

__global__ void __launch_bounds__(PERM_THREADS)
perm_fill_kernel(const int32_t* __restrict__ idx, int64_t NK, int ne, const int32_t* __restrict__ block_base,
                 int32_t* __restrict__ grouped) {
    constexpr int NW = PERM_THREADS / 32;
    __shared__ int cursor[MOE_MAX_NE];
    __shared__ int wcnt[NW][MOE_MAX_NE];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = threadIdx.x; e < ne; e += blockDim.x) cursor[e] = block_base[(int64_t)blockIdx.x * ne + e];
    const int64_t base = (int64_t)blockIdx.x * PERM_CHUNK;
    for (int it = 0; it < PERM_ITERS; ++it) {
        for (int i = threadIdx.x; i < NW * ne; i += blockDim.x) (&wcnt[0][0])[(i / ne) * MOE_MAX_NE + (i % ne)] = 0;
        __syncthreads();
        const int64_t s = base + it * PERM_THREADS + threadIdx.x;
        const bool live = s < NK;
        const int e = live ? idx[s] : -1 - lane;              // dead lanes match nobody
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        if (live && rank == 0) wcnt[warp][e] = __popc(peers);
        __syncthreads();
        if (live) {
            int pos = cursor[e] + rank;
            for (int w = 0; w < warp; ++w) pos += wcnt[w][e];
            grouped[pos] = (int32_t)s;
        }
        __syncthreads();
        for (int ee = threadIdx.x; ee < ne; ee += blockDim.x) {
            int add = 0;
#pragma unroll
            for (int w = 0; w < NW; ++w) add += wcnt[w][ee];
            cursor[ee] += add;
        }
        __syncthreads();
    }
}

// Up to PERM_CHUNK slots (a decode batch): the three steps and the inverse in one block -
// histogram, scan over the experts, the same ranked fill (cursor = the expert's offset).
__global__ void __launch_bounds__(PERM_THREADS)
perm_small_kernel(const int32_t* __restrict__ idx, int NK, int ne, int32_t* __restrict__ grouped,
                  int32_t* __restrict__ inv, int32_t* __restrict__ offsets) {
    constexpr int NW = PERM_THREADS / 32;
    __shared__ int cursor[MOE_MAX_NE + 1];
    __shared__ int wcnt[NW][MOE_MAX_NE];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = threadIdx.x; e <= ne; e += blockDim.x) cursor[e] = 0;
    __syncthreads();
    int mine[PERM_ITERS];
#pragma unroll
    for (int it = 0; it < PERM_ITERS; ++it) {
        const int s = it * PERM_THREADS + threadIdx.x;
        mine[it] = s < NK ? idx[s] : -1;
        if (s < NK) atomicAdd(&cursor[mine[it]], 1);
    }
    __syncthreads();
    if (warp == 0) {
        // exclusive scan of the counts, 32 experts at a time
        int run = 0;
        for (int e0 = 0; e0 <= ne; e0 += 32) {
            const int e = e0 + lane;
            const int c = e < ne ? cursor[e] : 0;
            int incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            if (e <= ne) {
                cursor[e] = run + incl - c;
                offsets[e] = run + incl - c;
            }
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < PERM_ITERS; ++it) {
        if (it * PERM_THREADS >= NK) break;                   // uniform
        for (int i = threadIdx.x; i < NW * MOE_MAX_NE; i += blockDim.x) (&wcnt[0][0])[i] = 0;
        __syncthreads();
        const int s = it * PERM_THREADS + threadIdx.x;
        const bool live = s < NK;
        const int e = live ? mine[it] : -1 - lane;            // dead lanes match nobody
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        if (live && rank == 0) wcnt[warp][e] = __popc(peers);
        __syncthreads();
        if (live) {
            int pos = cursor[e] + rank;
            for (int w = 0; w < warp; ++w) pos += wcnt[w][e];
            grouped[pos] = (int32_t)s;
            if (inv) inv[s] = pos;
        }
        __syncthreads();
        for (int ee = threadIdx.x; ee < ne; ee += blockDim.x) {
            int add = 0;
#pragma unroll
            for (int w = 0; w < NW; ++w) add += wcnt[w][ee];
            cursor[ee] += add;
        }
        __syncthreads();
    }
}

// grouped, offsets and (optionally) the inverse permutation in one launch when the slots fit one block.
int moe_permutation_inv(const int32_t* idx, int64_t NK, int ne, int32_t* grouped, int32_t* inv, int32_t* offsets) {
    B200_REQUIRE(idx && grouped && offsets, "moe_permutation: null pointer");
    B200_REQUIRE(ne > 0 && ne <= MOE_MAX_NE, "moe_permutation: ne out of range");
    if (NK < 0 || NK > PERM_CHUNK) return fail(B200_EUNSUPPORTED, "moe_permutation_inv: more slots than one block takes");
    perm_small_kernel<<<1, PERM_THREADS, 0, stream()>>>(idx, (int)NK, ne, grouped, inv, offsets);
    B200_LAUNCH_CHECK("perm_small_kernel");
    return B200_OK;
}
int moe_permutation_small_max() { return PERM_CHUNK; }

int moe_permutation(const int32_t* idx, int64_t NK, int ne, int32_t* grouped, int32_t* offsets) {
    B200_REQUIRE(idx && grouped && offsets, "moe_permutation: null pointer");
    B200_REQUIRE(ne > 0 && ne <= MOE_MAX_NE, "moe_permutation: ne out of range");
    B200_REQUIRE(NK >= 0 && NK < ((int64_t)1 << 31), "moe_permutation: slot count out of range");
    if (NK <= PERM_CHUNK) return moe_permutation_inv(idx, NK, ne, grouped, nullptr, offsets);     // one block does it all
    const int nblocks = (int)std::max<int64_t>(1, ceil_div64(NK, PERM_CHUNK));
    void* wsp;
    int rc = workspace(WS_PERM).ensure((size_t)nblocks * ne * sizeof(int32_t) + 256, &wsp);
    if (rc) return rc;
    int32_t* bc = static_cast<int32_t*>(wsp);
    perm_count_kernel<<<nblocks, PERM_THREADS, 0, stream()>>>(idx, NK, ne, bc);
    B200_LAUNCH_CHECK("perm_count_kernel");
    perm_scan_kernel<<<1, 320, 0, stream()>>>(bc, nblocks, ne, offsets);
    B200_LAUNCH_CHECK("perm_scan_kernel");
    perm_fill_kernel<<<nblocks, PERM_THREADS, 0, stream()>>>(idx, NK, ne, bc, grouped);
    B200_LAUNCH_CHECK("perm_fill_kernel");
    return B200_OK;
}

// ---------------------------------------------------------------------------
// Experts, token-major (small N): every (token, k) slot and every token's shared
// expert is an independent job.
//   kernel 1  act[job][i] = silu(gate_e[i].x_t) * up_e[i].x_t        (one warp per i)
//   kernel 2  out[t][j]   = shared_down[j].act_sh + sum_k w_k down_{e_k}[j].act_k
// ---------------------------------------------------------------------------
struct MoeArgs {
    const float* x;
    const uint8_t *gates, *ups, *downs, *sh_g, *sh_u, *sh_d;
    const int32_t* idx;     // [N,K]
    const float* w;         // [N,K]
    float* act;             // [N*K, E]
    float* sh_act;          // [N, SH]
    float *s_gate, *s_up;   // optional [N*K, E]
    float* out;             // [N, d]
    int N, d, E, ne, K, SH;
};

template <int KIND>
__global__ void __launch_bounds__(GEMV_THREADS) moe_gate_up_kernel(MoeArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = blockIdx.x * GEMV_WARPS + warp;
    const int job = blockIdx.y;
    const int routed = a.N * a.K;
    float g[1], u[1];
    if (job < routed) {
        if (i >= a.E) return;
        const int t = job / a.K, e = a.idx[job];
        const float* xt = a.x + (int64_t)t * a.d;
        gemv_row<KIND, 1>(xt, a.gates, (int64_t)e * a.E + i, 1, a.d, lane, g);
        gemv_row<KIND, 1>(xt, a.ups, (int64_t)e * a.E + i, 1, a.d, lane, u);
        if (lane == 0) {
            const int64_t o = (int64_t)job * a.E + i;
            a.act[o] = silu_acc(g[0]) * u[0];
            if (a.s_gate) a.s_gate[o] = g[0];
            if (a.s_up) a.s_up[o] = u[0];
        }
    } else {
        if (i >= a.SH) return;
        const int t = job - routed;
        const float* xt = a.x + (int64_t)t * a.d;
        gemv_row<KIND, 1>(xt, a.sh_g, i, 1, a.d, lane, g);
        gemv_row<KIND, 1>(xt, a.sh_u, i, 1, a.d, lane, u);
        if (lane == 0) a.sh_act[(int64_t)t * a.SH + i] = silu_acc(g[0]) * u[0];
    }
}

template <int KIND>
__global__ void __launch_bounds__(GEMV_THREADS) moe_down_combine_kernel(MoeArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.x * GEMV_WARPS + warp;
    const int t = blockIdx.y;
    if (j >= a.d) return;
    float r[1];
    float acc = 0.0f;
    if (a.sh_d) {
        gemv_row<KIND, 1>(a.sh_act + (int64_t)t * a.SH, a.sh_d, j, 1, a.SH, lane, r);
        acc = r[0];
    }
    for (int k = 0; k < a.K; ++k) {
        const int slot = t * a.K + k;
        const int e = a.idx[slot];
        gemv_row<KIND, 1>(a.act + (int64_t)slot * a.E, a.downs, (int64_t)e * a.d + j, 1, a.E, lane, r);
        acc = __fadd_rn(acc, __fmul_rn(a.w[slot], r[0]));
    }
    if (lane == 0) a.out[(int64_t)t * a.d + j] = acc;
}

template <int KIND>
static int launch_experts(const MoeArgs& a) {
    const bool shared = a.sh_g != nullptr;
    const int jobs = a.N * a.K + (shared ? a.N : 0);
    const int rows = std::max(a.E, shared ? a.SH : 0);
    moe_gate_up_kernel<KIND><<<dim3(ceil_div(rows, GEMV_WARPS), jobs), GEMV_THREADS, 0, stream()>>>(a);
    B200_LAUNCH_CHECK("moe_gate_up_kernel");
    moe_down_combine_kernel<KIND><<<dim3(ceil_div(a.d, GEMV_WARPS), a.N), GEMV_THREADS, 0, stream()>>>(a);
    B200_LAUNCH_CHECK("moe_down_combine_kernel");
    return B200_OK;
}

// ---------------------------------------------------------------------------
// Router for many tokens.  The logit of (token, expert) keeps the reference's
// sequential fp32 chain over groups of four, but the chains of a 32-token x
// 64-expert tile advance together: activations and router rows are staged in
// shared memory 64 columns at a time and every thread carries TPT x EPT chains in
// registers (4 x 2 for prompts; 1 x 1 for a batch of decode tokens, so that the few
// chains spread over many SMs).  A second kernel finishes each token with one warp.
// ---------------------------------------------------------------------------
constexpr int RT_K = 64, RT_LD = RT_K + 4;

template <int TPT, int EPT>
__global__ void __launch_bounds__(256)
route_logits_kernel(const float* __restrict__ x, const float* __restrict__ router_w, float* __restrict__ logits,
                    int64_t N, int d, int ne) {
    constexpr int RT_TOK = 8 * TPT, RT_EXP = 32 * EPT;
    __shared__ __align__(16) float xs[RT_TOK][RT_LD];
    __shared__ __align__(16) float ws[RT_EXP][RT_LD];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t t0 = (int64_t)blockIdx.x * RT_TOK;
    const int e0 = blockIdx.y * RT_EXP;
    float acc[TPT][EPT] = {};
    // The next 64 columns of the tile are fetched into registers while the current ones
    // are consumed from shared memory, so the global-memory latency of a chunk is paid
    // once, not once per chunk.
    constexpr int ITEMS = (RT_TOK + RT_EXP) * (RT_K / 4);
    constexpr int PER = (ITEMS + 255) / 256;
    float4 pre[PER];
    auto fetch = [&](int k0) {
        const int kc = min(RT_K, d - k0);
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int i = u * 256 + threadIdx.x;
            const int row = i / (RT_K / 4), c4 = (i % (RT_K / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < ITEMS && c4 < kc) {
                if (row < RT_TOK) {
                    if (t0 + row < N) v = *reinterpret_cast<const float4*>(x + (t0 + row) * d + k0 + c4);
                } else if (e0 + row - RT_TOK < ne) {
                    v = *reinterpret_cast<const float4*>(router_w + (int64_t)(e0 + row - RT_TOK) * d + k0 + c4);
                }
            }
            pre[u] = v;
        }
    };
    auto park = [&]() {
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int i = u * 256 + threadIdx.x;
            if (i < ITEMS) {
                const int row = i / (RT_K / 4), c4 = (i % (RT_K / 4)) * 4;
                float* dst = row < RT_TOK ? &xs[row][c4] : &ws[row - RT_TOK][c4];
                *reinterpret_cast<float4*>(dst) = pre[u];
            }
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < d; k0 += RT_K) {
        const int kc = min(RT_K, d - k0);              // a multiple of 4
        __syncthreads();                               // the previous chunk has been consumed
        park();
        __syncthreads();
        if (k0 + RT_K < d) fetch(k0 + RT_K);
        for (int g = 0; g < kc; g += 4) {
            float4 a[TPT], b[EPT];
#pragma unroll
            for (int i = 0; i < TPT; ++i) a[i] = *reinterpret_cast<const float4*>(&xs[TPT * ty + i][g]);
#pragma unroll
            for (int j = 0; j < EPT; ++j) b[j] = *reinterpret_cast<const float4*>(&ws[tx + 32 * j][g]);
#pragma unroll
            for (int i = 0; i < TPT; ++i)
#pragma unroll
                for (int j = 0; j < EPT; ++j) {
                    float s = __fadd_rn(__fmul_rn(a[i].x, b[j].x), __fmul_rn(a[i].y, b[j].y));
                    s = __fadd_rn(s, __fmul_rn(a[i].z, b[j].z));
                    s = __fadd_rn(s, __fmul_rn(a[i].w, b[j].w));
                    acc[i][j] = __fadd_rn(acc[i][j], s);
                }
        }
    }
#pragma unroll
    for (int i = 0; i < TPT; ++i)
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const int64_t t = t0 + TPT * ty + i;
            const int e = e0 + tx + 32 * j;
            if (t < N && e < ne) logits[t * ne + e] = acc[i][j];
        }
}

// A decode batch (tens of tokens): the tiled kernel above would occupy N / 8 x ne / 32 blocks -
// 16 SMs for 64 tokens - each crawling along 1536-long chains.  Here a block takes 8 tokens x 8
// experts (64 chains), and the two parts of a chain are split over its threads: the group sums
// ((a0 b0 + a1 b1) + a2 b2) + a3 b3 of a 1024-column piece are independent and go to shared
// memory four threads per chain; one thread per chain then adds them in order (the only
// sequential part: one dependent add per group).  Same values, same order as the chains above.
constexpr int RC_TOK = 8, RC_EXP = 8, RC_COLS = 1024, RC_LD = RC_COLS + 4, RC_GLD = RC_COLS / 4 + 1;
constexpr size_t RC_SMEM = ((size_t)(RC_TOK + RC_EXP) * RC_LD + (size_t)RC_TOK * RC_EXP * RC_GLD) * 4;
__global__ void __launch_bounds__(256)
route_logits_chains_kernel(const float* __restrict__ x, const float* __restrict__ router_w, float* __restrict__ logits,
                           int64_t N, int d, int ne, const float* __restrict__ router_bias, float* __restrict__ probs_out,
                           int32_t* __restrict__ idx_out, float* __restrict__ w_out, int K, int* __restrict__ counters) {
    extern __shared__ __align__(16) float rc_smem[];
    float* xs = rc_smem;                                  // [RC_TOK][RC_LD]
    float* ws = xs + RC_TOK * RC_LD;                      // [RC_EXP][RC_LD]
    float* gs = ws + RC_EXP * RC_LD;                      // [64 chains][RC_GLD]
    const int64_t t0 = (int64_t)blockIdx.x * RC_TOK;
    const int e0 = blockIdx.y * RC_EXP;
    const int c = threadIdx.x & 63, sub = threadIdx.x >> 6;          // chain, which quarter of its groups
    const int tc = c & 7, ec = c >> 3;
    float chain = 0.0f;
    // A piece is at most 256 runs of four wide: one run per thread and row, all 16 loads in flight;
    // the next piece is fetched into registers while the current one is worked on.
    const int q = threadIdx.x, c4 = q * 4;
    float4 v[RC_TOK + RC_EXP];
    auto fetch = [&](int k0) {
        const int q4 = min(RC_COLS, d - k0) >> 2;
#pragma unroll
        for (int row = 0; row < RC_TOK + RC_EXP; ++row) {
            v[row] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (q < q4) {
                if (row < RC_TOK) {
                    if (t0 + row < N) v[row] = *reinterpret_cast<const float4*>(x + (t0 + row) * d + k0 + c4);
                } else if (e0 + row - RC_TOK < ne) {
                    v[row] = *reinterpret_cast<const float4*>(router_w + (int64_t)(e0 + row - RC_TOK) * d + k0 + c4);
                }
            }
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < d; k0 += RC_COLS) {
        const int kc = min(RC_COLS, d - k0), q4 = kc >> 2;           // kc % 4 == 0
        __syncthreads();                                             // the previous piece has been consumed
        if (q < q4) {
#pragma unroll
            for (int row = 0; row < RC_TOK + RC_EXP; ++row)
                *reinterpret_cast<float4*>((row < RC_TOK ? xs + row * RC_LD : ws + (row - RC_TOK) * RC_LD) + c4) = v[row];
        }
        __syncthreads();
        if (k0 + RC_COLS < d) fetch(k0 + RC_COLS);
        const float* xa = xs + tc * RC_LD;
        const float* wb = ws + ec * RC_LD;
        float* gc = gs + c * RC_GLD;
#pragma unroll 4
        for (int g = sub; g < q4; g += 4) {
            const float4 a = *reinterpret_cast<const float4*>(xa + 4 * g);
            const float4 b = *reinterpret_cast<const float4*>(wb + 4 * g);
            float t = __fadd_rn(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y));
            t = __fadd_rn(t, __fmul_rn(a.z, b.z));
            t = __fadd_rn(t, __fmul_rn(a.w, b.w));
            gc[g] = t;
        }
        __syncthreads();
        if (threadIdx.x < 64) {
#pragma unroll 8
            for (int g = 0; g < q4; ++g) chain = __fadd_rn(chain, gc[g]);
        }
    }
    if (threadIdx.x < 64) {
        const int64_t t = t0 + tc;
        const int e = e0 + ec;
        if (t < N && e < ne) logits[t * ne + e] = chain;
    }
    // The block that completes a token group's last expert tile turns the group's logits into
    // (idx, w), one warp per token: nobody waits - each block counts itself in after publishing
    // its logits, and whoever counts last finds all of them (fence before the count and after it).
    __shared__ int s_last;
    if (!counters) return;                                   // the caller finishes with route_finish_kernel
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&counters[blockIdx.x], 1) == (int)gridDim.y - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        float* s_p = rc_smem + (size_t)warp * (2 * MOE_MAX_NE + 2 * MOE_MAX_K);      // the tiles are dead
        float* s_sel = s_p + MOE_MAX_NE;
        float* s_w = s_sel + MOE_MAX_NE;
        int* s_idx = reinterpret_cast<int*>(s_w + MOE_MAX_K);
        const int64_t t = t0 + warp;
        if (warp < RC_TOK && t < N) {
            route_finish_warp(logits + t * ne, router_bias, ne, K, s_p, s_sel, s_idx, s_w,
                              probs_out ? probs_out + t * ne : nullptr, lane);
            if (lane < K) {
                idx_out[t * K + lane] = s_idx[lane];
                w_out[t * K + lane] = s_w[lane];
            }
        }
        if (threadIdx.x == 0) counters[blockIdx.x] = 0;       // ready for the next call
    }
}

// Arrival counters of the kernel above (one per token group), zeroed once; every call leaves them zero.
// Not created while the stream is being captured into a graph (an allocation and a memset on the
// default stream do not belong there): the caller then runs the separate finishing kernel.
static int* route_counters() {
    static int* p = nullptr;
    if (!p) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream(), &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
            cudaGetLastError();
            return nullptr;
        }
        if (cudaMalloc(&p, 4096) != cudaSuccess) { p = nullptr; cudaGetLastError(); return nullptr; }
        if (cudaMemset(p, 0, 4096) != cudaSuccess) { cudaFree(p); p = nullptr; cudaGetLastError(); return nullptr; }
    }
    return p;
}

constexpr int RF_WARPS = 8;
__global__ void __launch_bounds__(RF_WARPS * 32)
route_finish_kernel(const float* __restrict__ logits, const float* __restrict__ router_bias, float* __restrict__ probs_out,
                    int32_t* __restrict__ idx_out, float* __restrict__ w_out, int64_t N, int ne, int K) {
    __shared__ float s_p[RF_WARPS][MOE_MAX_NE], s_sel[RF_WARPS][MOE_MAX_NE], s_w[RF_WARPS][MOE_MAX_K];
    __shared__ int s_idx[RF_WARPS][MOE_MAX_K];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * RF_WARPS + warp;
    if (t >= N) return;
    route_finish_warp(logits + t * ne, router_bias, ne, K, s_p[warp], s_sel[warp], s_idx[warp], s_w[warp],
                      probs_out ? probs_out + t * ne : nullptr, lane);
    if (lane < K) {
        idx_out[t * K + lane] = s_idx[warp][lane];
        w_out[t * K + lane] = s_w[warp][lane];
    }
}

int moe_route(const float* x, const float* router_w, const float* router_bias, float* probs,
              int32_t* idx, float* w, int64_t N, int d, int ne, int K) {
    if (N >= 16 && d % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        void* wsp;
        int rc = workspace(WS_ROUTE).ensure((size_t)N * ne * 4 + 256, &wsp);
        if (rc) return rc;
        float* logits = static_cast<float*>(wsp);
        if (N <= 256) {
            static bool configured = false;
            if (!configured) {
                B200_CUDA(cudaFuncSetAttribute(route_logits_chains_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)RC_SMEM));
                configured = true;
            }
            int* counters = route_counters();
            const dim3 grid((unsigned)ceil_div64(N, RC_TOK), ceil_div(ne, RC_EXP));
            route_logits_chains_kernel<<<grid, 256, RC_SMEM, stream()>>>(x, router_w, logits, N, d, ne, router_bias, probs, idx,
                                                                         w, K, counters);
            B200_LAUNCH_CHECK("route_logits_chains_kernel");
            if (counters) return B200_OK;
        } else if (N <= 1024) {
            const dim3 grid((unsigned)ceil_div64(N, 8), ceil_div(ne, 32));
            route_logits_kernel<1, 1><<<grid, 256, 0, stream()>>>(x, router_w, logits, N, d, ne);
        } else {
            // 32 tokens x 32 experts per block: twice the blocks of a 32 x 64 tile, which
            // measured 15 % faster at 4096 tokens x 64 experts (more resident warps per SM)
            const dim3 grid((unsigned)ceil_div64(N, 32), ceil_div(ne, 32));
            route_logits_kernel<4, 1><<<grid, 256, 0, stream()>>>(x, router_w, logits, N, d, ne);
        }
        B200_LAUNCH_CHECK("route_logits_kernel");
        route_finish_kernel<<<(unsigned)ceil_div64(N, RF_WARPS), RF_WARPS * 32, 0, stream()>>>(logits, router_bias, probs,
                                                                                                  idx, w, N, ne, K);
        B200_LAUNCH_CHECK("route_finish_kernel");
        return B200_OK;
    }
    // shared memory: x + as many group rows as fit in ~96 KB
    const int groups = d >> 2;
    const size_t x_bytes = (size_t)((d + 3) & ~3) * 4;
    int chunk = (int)std::min<size_t>((size_t)std::max(groups, 1), (96 * 1024 - x_bytes) / ((size_t)(ne + 1) * 4));
    B200_REQUIRE(chunk >= 1, "moe: hidden size too large for the router kernel");
    const size_t smem = x_bytes + (size_t)chunk * (ne + 1) * 4;
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        B200_CUDA(cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        configured = 100 * 1024;
    }
    moe_route_kernel<<<(unsigned)N, ROUTE_THREADS, smem, stream()>>>(x, router_w, router_bias, probs, idx, w, d, ne,
                                                                     K, chunk);
    B200_LAUNCH_CHECK("moe_route_kernel");
    return B200_OK;
}

// kind: template tag.  Weight pointers are raw bytes in that kind.
int moe_forward(const float* x, const float* router_w, const float* router_bias, const void* gates,
                const void* ups, const void* downs, const void* sh_g, const void* sh_u, const void* sh_d,
                float* out, float* probs_cache, int32_t* idx_cache, float* w_cache, float* s_gate,
                float* s_up, float* s_act, int64_t N, int d, int E, int ne, int K, int SH, int kind) {
    if (N <= 0) return B200_OK;
    B200_REQUIRE(K >= 1 && K <= MOE_MAX_K, "moe_forward: K must be in [1,%d]", MOE_MAX_K);
    B200_REQUIRE(ne > 0 && ne <= MOE_MAX_NE && K <= ne, "moe_forward: ne out of range");
    B200_REQUIRE(d > 0 && E > 0, "moe_forward: bad dims");
    B200_REQUIRE(x && router_w && gates && ups && downs && out, "moe_forward: null pointer");
    B200_REQUIRE(d % 32 == 0 && E % 32 == 0, "moe_forward: d and E must be multiples of 32");
    B200_REQUIRE((reinterpret_cast<uintptr_t>(router_w) & 15) == 0 && d % 4 == 0, "moe_forward: router_w alignment");
    const bool shared = sh_g && sh_u && sh_d;
    if (shared) B200_REQUIRE(SH > 0 && SH % 32 == 0, "moe_forward: SH must be a positive multiple of 32");
    if (kind >= 0 && kind <= 3)
        B200_REQUIRE(d % q_block_elems(kind) == 0 && E % q_block_elems(kind) == 0 &&
                         (!shared || SH % q_block_elems(kind) == 0),
                     "moe_forward: d, E and SH must be multiples of the quantisation block");
    B200_REQUIRE(N * K < ((int64_t)1 << 31), "moe_forward: N too large");

    // Many tokens over fp16 / packed experts: expert-grouped tensor-core GEMMs.  The
    // optional fp32 scratch outputs only exist on the token-major path.
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    // A decode batch: at most MOE_UNITS_MAX_ROWS rows per expert on average.  The experts'
    // rows would leave the 128-row tensor-core tiles nearly empty; they run as weight streams
    // shared by their tokens instead (moe_units.cu).
    if (N > 8 && N * K <= (int64_t)MOE_UNITS_MAX_ROWS * ne && kind != KIND_F32 && !s_gate && !s_up && !s_act && aligned16(x) &&
        aligned16(out) && aligned16(gates) && aligned16(ups) && aligned16(downs) && d % 8 == 0 &&
        (kind != 3 || (d % 256 == 0 && E % 256 == 0)) && ne <= 256 &&
        (!shared || (aligned16(sh_g) && aligned16(sh_u) && aligned16(sh_d) && (kind == KIND_F16 || SH % 256 == 0)))) {
        const int rc = moe_forward_units(x, router_w, router_bias, gates, ups, downs, sh_g, sh_u, sh_d, out, probs_cache,
                                         idx_cache, w_cache, N, d, E, ne, K, shared ? SH : 0, kind);
        if (rc != B200_EUNSUPPORTED) return rc;
    }
    if (N >= GEMM_MIN_ROWS && kind != KIND_F32 && !s_gate && !s_up && !s_act && aligned16(x) && aligned16(out) &&
        aligned16(gates) && aligned16(ups) && aligned16(downs) &&
        (!shared || (aligned16(sh_g) && aligned16(sh_u) && aligned16(sh_d))))
        return moe_forward_grouped(x, router_w, router_bias, gates, ups, downs, sh_g, sh_u, sh_d, out, probs_cache,
                                   idx_cache, w_cache, N, d, E, ne, K, shared ? SH : 0, kind);

    // workspace: idx | w | act | sh_act
    const size_t NK = (size_t)N * K;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off += (bytes + 255) & ~(size_t)255; return o; };
    const size_t o_idx = take(NK * 4), o_w = take(NK * 4);
    const size_t o_act = s_act ? 0 : take(NK * E * 4);
    const size_t o_sh = shared ? take((size_t)N * SH * 4) : 0;
    void* wsp;
    int rc = workspace(WS_MOE).ensure(off + 256, &wsp);
    if (rc) return rc;
    char* base = static_cast<char*>(wsp);
    int32_t* idx = idx_cache ? idx_cache : reinterpret_cast<int32_t*>(base + o_idx);
    float* w = w_cache ? w_cache : reinterpret_cast<float*>(base + o_w);

    rc = moe_route(x, router_w, router_bias, probs_cache, idx, w, N, d, ne, K);
    if (rc) return rc;

    MoeArgs a;
    a.x = x;
    a.gates = static_cast<const uint8_t*>(gates);
    a.ups = static_cast<const uint8_t*>(ups);
    a.downs = static_cast<const uint8_t*>(downs);
    a.sh_g = shared ? static_cast<const uint8_t*>(sh_g) : nullptr;
    a.sh_u = shared ? static_cast<const uint8_t*>(sh_u) : nullptr;
    a.sh_d = shared ? static_cast<const uint8_t*>(sh_d) : nullptr;
    a.idx = idx;
    a.w = w;
    a.act = s_act ? s_act : reinterpret_cast<float*>(base + o_act);
    a.sh_act = shared ? reinterpret_cast<float*>(base + o_sh) : nullptr;
    a.s_gate = s_gate;
    a.s_up = s_up;
    a.out = out;
    a.N = (int)N; a.d = d; a.E = E; a.ne = ne; a.K = K; a.SH = shared ? SH : 0;
    // grid.y carries the jobs: walk the tokens in chunks that keep it under 65535
    const int chunk_tokens = std::max(1, 65535 / (K + 1));
    for (int64_t t0 = 0; t0 < N; t0 += chunk_tokens) {
        MoeArgs c = a;
        c.N = (int)std::min<int64_t>(chunk_tokens, N - t0);
        c.x = a.x + t0 * d;
        c.idx = a.idx + t0 * K;
        c.w = a.w + t0 * K;
        c.act = a.act + t0 * K * E;
        if (a.sh_act) c.sh_act = a.sh_act + t0 * SH;
        if (a.s_gate) c.s_gate = a.s_gate + t0 * K * E;
        if (a.s_up) c.s_up = a.s_up + t0 * K * E;
        c.out = a.out + t0 * d;
        switch (kind) {
            case 0: rc = launch_experts<0>(c); break;
            case 1: rc = launch_experts<1>(c); break;
            case 2: rc = launch_experts<2>(c); break;
            case 3: rc = launch_experts<3>(c); break;
            case KIND_F16: rc = launch_experts<KIND_F16>(c); break;
            default: rc = launch_experts<KIND_F32>(c); break;
        }
        if (rc) return rc;
    }
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_moe_forward(const float* x, const float* router_w, const float* gates, const float* ups,
                     const float* downs, const float* sh_g, const float* sh_u, const float* sh_d,
                     float* out, float* probs_cache, int32_t* idx_cache, float* w_cache,
                     float* s_gate, float* s_up, float* s_act,
                     int64_t N, int d, int E, int ne, int K, int SH) {
    return moe_forward(x, router_w, nullptr, gates, ups, downs, sh_g, sh_u, sh_d, out, probs_cache, idx_cache,
                       w_cache, s_gate, s_up, s_act, N, d, E, ne, K, SH, KIND_F32);
}
int b200_moe_forward_bias(const float* x, const float* router_w, const float* router_bias,
                          const float* gates, const float* ups, const float* downs,
                          const float* sh_g, const float* sh_u, const float* sh_d,
                          float* out, float* probs_cache, int32_t* idx_cache, float* w_cache,
                          float* s_gate, float* s_up, float* s_act,
                          int64_t N, int d, int E, int ne, int K, int SH) {
    return moe_forward(x, router_w, router_bias, gates, ups, downs, sh_g, sh_u, sh_d, out, probs_cache, idx_cache,
                       w_cache, s_gate, s_up, s_act, N, d, E, ne, K, SH, KIND_F32);
}
int b200_moe_forward_half(const float* x, const float* router_w, const uint16_t* gates,
                          const uint16_t* ups, const uint16_t* downs, const uint16_t* sh_g,
                          const uint16_t* sh_u, const uint16_t* sh_d, float* out,
                          float* probs_cache, int32_t* idx_cache, float* w_cache,
                          float* s_gate, float* s_up, float* s_act,
                          int64_t N, int d, int E, int ne, int K, int SH, int qkind) {
    B200_REQUIRE(qkind >= -1 && qkind <= 3, "moe_forward_half: unknown qkind %d", qkind);
    return moe_forward(x, router_w, nullptr, gates, ups, downs, sh_g, sh_u, sh_d, out, probs_cache, idx_cache,
                       w_cache, s_gate, s_up, s_act, N, d, E, ne, K, SH, tag_of_qkind(qkind));
}
int b200_moe_forward_bias_half(const float* x, const float* router_w, const float* router_bias,
                               const uint16_t* gates, const uint16_t* ups, const uint16_t* downs,
                               const uint16_t* sh_g, const uint16_t* sh_u, const uint16_t* sh_d,
                               float* out, float* probs_cache, int32_t* idx_cache, float* w_cache,
                               float* s_gate, float* s_up, float* s_act,
                               int64_t N, int d, int E, int ne, int K, int SH, int qkind) {
    B200_REQUIRE(qkind >= -1 && qkind <= 3, "moe_forward_bias_half: unknown qkind %d", qkind);
    return moe_forward(x, router_w, router_bias, gates, ups, downs, sh_g, sh_u, sh_d, out, probs_cache, idx_cache,
                       w_cache, s_gate, s_up, s_act, N, d, E, ne, K, SH, tag_of_qkind(qkind));
}
int b200_moe_permutation(const int32_t* idx, int64_t NK, int ne, int32_t* grouped, int32_t* offsets) {
    return moe_permutation(idx, NK, ne, grouped, offsets);
}

}  // extern "C"
