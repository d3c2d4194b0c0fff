// Fused decode-step kernels (a few tokens per step): every weight matrix is streamed
// once through a shared-memory ring by the TMA unit while the math runs out of
// shared memory; the RMSNorm before a projection is that kernel's prologue, the
// Mamba conv step / the residual add its epilogue; the MoE layer is three such
// kernels (router logits + shared expert, routed gate/up, down + combine).
//
// These fuse across the reference's op boundaries (rmsnorm_forward -> linear ->
// add_inplace in Generator::decode_step_logits, inference/generator.cpp:253-436),
// so they are reached only through the decoder's fused mode; the per-op C ABI keeps
// the reference's granularity.
//
// All kernels here are launched with programmatic dependent launch: work that does
// not depend on the previous kernel (barrier set-up, weight streaming, parameter
// prefetch) runs before griddepcontrol.wait and overlaps the predecessor's tail.
#include "fused.cuh"

namespace b200 {

static int* g_status_dev = nullptr;
int* stream_status_ptr() {
    if (!g_status_dev) {
        if (cudaMalloc(&g_status_dev, 256) != cudaSuccess) return nullptr;
        cudaMemset(g_status_dev, 0, 256);
    }
    return g_status_dev;
}
int stream_status_check(const char* who) {
    if (!g_status_dev) return B200_OK;
    int h = 0;
    B200_CUDA(cudaMemcpy(&h, g_status_dev, 4, cudaMemcpyDeviceToHost));
    if (h != 0) {
        cudaMemset(g_status_dev, 0, 4);
        return fail(B200_ECUDA, "%s: a bounded wait inside a streaming kernel ran out (status %d)", who, h);
    }
    return B200_OK;
}

constexpr int SG_CONSUMERS = 4;                    // consumer warps
constexpr int SG_CTHREADS = SG_CONSUMERS * 32;
constexpr int SG_THREADS = SG_CTHREADS + 32;       // + one producer warp
constexpr int SG_MAX_STAGES = 4;
constexpr int SMEM_BUDGET = 150 * 1024;            // per CTA, leaves room for a second CTA / the next kernel

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(SG_CTHREADS) : "memory"); }

// Sum over the consumer threads (0..127); result in every consumer thread.
__device__ __forceinline__ double consumer_sum_d(double v, double* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    v = warp_sum_d(v);
    consumer_sync();
    if (lane == 0) red[wid] = v;
    consumer_sync();
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < SG_CONSUMERS; ++w) t += red[w];
    return t;
}

// The shared-memory ring.
struct Ring {
    uint8_t* stages;
    uint64_t *full, *empty;
    int stage_bytes, n_stages;
    int* status;
    __device__ __forceinline__ void init() {
        if (threadIdx.x == 0) {
            for (int s = 0; s < n_stages; ++s) {
                mbar_init(&full[s], 1);
                mbar_init(&empty[s], SG_CONSUMERS);
            }
            mbar_fence_init();
        }
        __syncthreads();
    }
    __device__ __forceinline__ uint8_t* stage(int i) const { return stages + (size_t)(i % n_stages) * stage_bytes; }
    // producer side
    __device__ __forceinline__ bool acquire(int i) {
        return i < n_stages || mbar_wait(&empty[i % n_stages], ((i / n_stages) - 1) & 1, status);
    }
    __device__ __forceinline__ void expect(int i, uint32_t bytes) { mbar_expect_tx(&full[i % n_stages], bytes); }
    __device__ __forceinline__ void copy(int i, int offset, const void* src, uint32_t bytes) {
        tma_load_1d(stage(i) + offset, src, bytes, &full[i % n_stages]);
    }
    // never leave with copies of this CTA still in flight
    __device__ __forceinline__ void drain(int issued) {
        for (int i = max(0, issued - n_stages); i < issued; ++i)
            if (!mbar_wait(&full[i % n_stages], (i / n_stages) & 1, status)) break;
    }
    // consumer side
    __device__ __forceinline__ bool wait_full(int i) { return mbar_wait(&full[i % n_stages], (i / n_stages) & 1, status); }
    __device__ __forceinline__ void release(int i) {
        __syncwarp();
        if ((threadIdx.x & 31) == 0) mbar_arrive(&empty[i % n_stages]);
    }
};

// Activations of one token into shared memory (unit-major), optionally RMS-normed:
// xs[k] = x[k] * inv * norm_w[k] in the reference's operand order
// (core/math_cpu.cpp:299-316, inv from a double sum of squares).  nw_s is norm_w
// prefetched into shared memory before the dependency wait.  Consumer threads only.
template <int KIND, bool RMS>
__device__ __forceinline__ void stage_x(const float* __restrict__ x, const float* nw_s, float* xs, int K, float eps,
                                        double* red) {
    double ss = 0.0;
    for (int k = threadIdx.x; k < K; k += SG_CTHREADS) {
        const float v = x[k];
        xs[xs_index<KIND>(k)] = v;
        if (RMS) ss += (double)v * v;
    }
    if (RMS) {
        ss = consumer_sum_d(ss, red);
        const double inv_d = 1.0 / sqrt(ss / (double)K + (double)eps);
        const float inv = isfinite(inv_d) ? (float)inv_d : 0.0f;
        for (int k = threadIdx.x; k < K; k += SG_CTHREADS) {
            const int i = xs_index<KIND>(k);
            xs[i] = xs[i] * inv * nw_s[k];
        }
    }
}

// ===========================================================================
// 1. single-matrix streamed GEMV
// ===========================================================================
template <int KIND, int MT, int PRO, int EPI>
__global__ void __launch_bounds__(SG_THREADS) stream_gemv_kernel(SgArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    Ring ring;
    ring.stages = smem;
    ring.stage_bytes = a.stage_bytes;
    ring.n_stages = a.n_stages;
    ring.status = a.status;
    float* xs = reinterpret_cast<float*>(smem + (size_t)a.n_stages * a.stage_bytes);
    const int xs_tok = xs_floats(a.K);
    float* nw_s = xs + (size_t)MT * xs_tok;                       // [K] when PRO_RMS
    ring.full = reinterpret_cast<uint64_t*>(nw_s + (PRO == PRO_RMS ? a.K : 0));
    ring.empty = ring.full + SG_MAX_STAGES;
    double* red = reinterpret_cast<double*>(ring.empty + SG_MAX_STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first = blockIdx.x, step = gridDim.x;
    const int n_my = first < a.num_tiles ? (a.num_tiles - first + step - 1) / step : 0;
    ring.init();
    if (threadIdx.x == 0) pdl_launch_dependents();

    if (warp == SG_CONSUMERS) {
        // producer: the weights do not depend on the previous kernel - start at once
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < n_my; ++i) {
                if (!ring.acquire(i)) break;
                const int tile = first + i * step;
                const int rows = min(a.rows_per_tile, a.N - tile * a.rows_per_tile);
                const uint32_t bytes = (uint32_t)(rows * a.row_bytes);
                ring.expect(i, bytes);
                ring.copy(i, 0, a.w + (int64_t)tile * a.rows_per_tile * a.row_bytes, bytes);
                issued = i + 1;
            }
            ring.drain(issued);
        }
        return;
    }

    // consumers
    if (PRO == PRO_RMS)
        for (int k = threadIdx.x; k < a.K; k += SG_CTHREADS) nw_s[k] = a.norm_w[k];
    pdl_wait();
    for (int m = 0; m < a.M; ++m)
        stage_x<KIND, PRO == PRO_RMS>(a.x + (int64_t)m * a.x_stride, nw_s, xs + m * xs_tok, a.K, a.eps, red);
    float in_scale = 1.0f;            // lane m holds token m's scale
    if (a.in_partials) {
        // gated-norm statistic: inv = 1/sqrt(mean + eps) from block partial sums (fixed order)
        for (int m = 0; m < a.M; ++m) {
            double t = 0.0;
            for (int i = threadIdx.x; i < a.n_partials; i += SG_CTHREADS) t += a.in_partials[(int64_t)m * a.n_partials + i];
            t = consumer_sum_d(t, red) / (double)a.in_dim;
            if (lane == m) in_scale = 1.0f / sqrtf((float)t + a.eps);
        }
    }
    consumer_sync();

    for (int i = 0; i < n_my; ++i) {
        const int tile = first + i * step;
        const int rows = min(a.rows_per_tile, a.N - tile * a.rows_per_tile);
        // epilogue operands are fetched before the dot product so their latency hides
        // (one row per warp per pass; lane m serves token m)
        if (!ring.wait_full(i)) break;
        const uint8_t* tile_smem = ring.stage(i);
        for (int r = warp; r < rows; r += SG_CONSUMERS) {
            const int n = tile * a.rows_per_tile + r;
            const bool owner = lane < MT && lane < a.M;
            float pre = 0.0f, st[4] = {0, 0, 0, 0}, wc[5] = {0, 0, 0, 0, 0};
            float* dst = nullptr;
            const bool is_conv = EPI == EPI_INPROJ && n >= a.p.d_inner && n < a.p.d_inner + a.p.conv_dim;
            if (owner) {
                if (EPI == EPI_RESIDUAL) {
                    dst = a.resid + (int64_t)lane * a.y_stride + n;
                    pre = *dst;
                } else if (is_conv && a.p.k <= 5) {
                    const int c = n - a.p.d_inner, win = a.p.k - 1;
                    const float* sp = a.conv_state + ((int64_t)lane * a.p.conv_dim + c) * win;
                    const float* wp = a.conv_w + (int64_t)c * a.p.k;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (j < win) st[j] = sp[j];
#pragma unroll
                    for (int j = 0; j < 5; ++j)
                        if (j < a.p.k) wc[j] = wp[j];
                    pre = a.conv_b ? a.conv_b[c] : 0.0f;
                }
            }
            float acc[MT];
            row_dot_xs<KIND, MT>(tile_smem + (int64_t)r * a.row_bytes, xs, xs_tok, a.M, a.K, lane, acc);
            if (owner) {
                float v = 0.0f;
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m == lane) v = acc[m];
                const int m = lane;
                v *= in_scale;
                if (EPI == EPI_STORE) {
                    a.y[(int64_t)m * a.y_stride + n] = v * a.out_scale;
                } else if (EPI == EPI_RESIDUAL) {
                    *dst = pre + v * a.res_mult;
                } else {
                    const MambaDims& p = a.p;
                    if (n < p.d_inner) {
                        a.gate[(int64_t)m * p.d_inner + n] = v;
                    } else if (is_conv) {
                        const int c = n - p.d_inner, win = p.k - 1;
                        float* sp = a.conv_state + ((int64_t)m * p.conv_dim + c) * win;
                        float t;
                        if (p.k <= 5) {
                            // window of raw inputs, oldest first; unfused ops in the reference's order
                            t = pre;
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (j < win) {
                                    t = __fadd_rn(t, __fmul_rn(wc[j], st[j]));
                                    if (j > 0) sp[j - 1] = st[j];
                                }
                            float wl = wc[0];
#pragma unroll
                            for (int j = 1; j < 5; ++j)
                                if (j == win) wl = wc[j];
                            t = __fadd_rn(t, __fmul_rn(wl, v));
                        } else {
                            const float* wp = a.conv_w + (int64_t)c * p.k;
                            t = a.conv_b ? a.conv_b[c] : 0.0f;
                            for (int j = 0; j < win; ++j) {
                                const float sv = sp[j];
                                t = __fadd_rn(t, __fmul_rn(wp[j], sv));
                                if (j > 0) sp[j - 1] = sv;
                            }
                            t = __fadd_rn(t, __fmul_rn(wp[win], v));
                        }
                        if (win > 0) sp[win - 1] = v;
                        a.bc[(int64_t)m * p.conv_dim + c] = silu_acc(t);
                    } else {
                        a.dt_raw[(int64_t)m * p.n_heads + (n - p.d_inner - p.conv_dim)] = v;
                    }
                }
            }
        }
        ring.release(i);
    }
}

// ===========================================================================
// 2. Mamba-2 state update (decode) + gated-norm statistics
// ===========================================================================
// grid (rows / FS_WARPS, batch); one warp per state row.  Writes u = y * silu(gate)
// * norm_w and one double partial sum of (y*silu(gate))^2 per block; the
// out-projection turns the partials into inv = 1/sqrt(mean + eps) and computes
// inv * (W u) - algebraically the reference's rmsnorm(y*silu(gate))*norm_w -> W.
constexpr int FS_WARPS = 8;
__global__ void __launch_bounds__(FS_WARPS * 32)
mamba_scan_norm_kernel(const float* __restrict__ bc, const float* __restrict__ dt_raw,
                       const float* __restrict__ gate, const float* __restrict__ dt_bias,
                       const float* __restrict__ a_log, const float* __restrict__ Dv,
                       const float* __restrict__ norm_w, float* __restrict__ ssm_state,
                       float* __restrict__ u_out, double* __restrict__ partials, MambaDims p) {
    __shared__ double wsum[FS_WARPS];
    if (threadIdx.x == 0) pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows = p.n_heads * p.d_head;
    const int row = blockIdx.x * FS_WARPS + warp;
    const int m = blockIdx.y;
    const bool live = row < rows;
    const bool vec = (p.d_state == 128);
    const int h = live ? row / p.d_head : 0;
    float* s = ssm_state + ((int64_t)m * rows + (live ? row : 0)) * p.d_state;
    // everything that does not depend on this token's projection: before the wait
    float4 sv = make_float4(0, 0, 0, 0);
    if (live && vec) sv = *reinterpret_cast<const float4*>(s + lane * 4);
    const float dtb = dt_bias[h], al = a_log[h], dsk = Dv[h];
    const float nw = live ? norm_w[row] : 0.0f;
    pdl_wait();
    double sq = 0.0;
    if (live) {
        const float* bcm = bc + (int64_t)m * p.conv_dim;
        const float xv = bcm[row];
        const float gt = gate[(int64_t)m * p.d_inner + row];
        const float uu = dt_raw[(int64_t)m * p.n_heads + h] + dtb;
        const float* Bv = bcm + p.d_inner;
        const float* Cv = Bv + p.d_state;
        float acc = 0.0f;
        float4 b4 = make_float4(0, 0, 0, 0), c4 = b4;
        if (vec) {
            b4 = *reinterpret_cast<const float4*>(Bv + lane * 4);
            c4 = *reinterpret_cast<const float4*>(Cv + lane * 4);
        }
        const float dt = (uu > 20.0f) ? uu : log1pf(expf(uu));
        const float A = -expf(al);
        const float dA = expf(__fmul_rn(A, dt));
        if (vec) {
            sv.x = __fadd_rn(__fmul_rn(dA, sv.x), __fmul_rn(__fmul_rn(dt, b4.x), xv));
            sv.y = __fadd_rn(__fmul_rn(dA, sv.y), __fmul_rn(__fmul_rn(dt, b4.y), xv));
            sv.z = __fadd_rn(__fmul_rn(dA, sv.z), __fmul_rn(__fmul_rn(dt, b4.z), xv));
            sv.w = __fadd_rn(__fmul_rn(dA, sv.w), __fmul_rn(__fmul_rn(dt, b4.w), xv));
            *reinterpret_cast<float4*>(s + lane * 4) = sv;
            acc = c4.x * sv.x + c4.y * sv.y + c4.z * sv.z + c4.w * sv.w;
        } else {
            for (int j = lane; j < p.d_state; j += 32) {
                const float sn = __fadd_rn(__fmul_rn(dA, s[j]), __fmul_rn(__fmul_rn(dt, Bv[j]), xv));
                s[j] = sn;
                acc += Cv[j] * sn;
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            const float y = acc + dsk * xv;
            const float v = y * silu_acc(gt);
            u_out[(int64_t)m * p.d_inner + row] = v * nw;
            sq = (double)v * v;
        }
    }
    if (lane == 0) wsum[warp] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < FS_WARPS; ++w) t += wsum[w];
        partials[(int64_t)m * gridDim.x + blockIdx.x] = t;
    }
}

// ===========================================================================
// 3. MoE layer in three streamed kernels
// ===========================================================================
// Router logit of one expert for one token, exactly as core/moe_cpu.cpp:76-83:
// group sums ((a0b0 + a1b1) + a2b2) + a3b3 by all lanes, then lane 0 adds them in
// order.  wrow: the expert's fp32 router row (shared memory); xs: the normed token
// in unit-major layout of weight kind KIND; gs: per-warp scratch of d/4 floats.
template <int KIND>
__device__ __forceinline__ float router_logit(const float* wrow, const float* xs, float* gs, int d, int lane) {
    const int groups = d >> 2;
    for (int g = lane; g < groups; g += 32) {
        const float4 b = *reinterpret_cast<const float4*>(wrow + 4 * g);
        const float4 a = *reinterpret_cast<const float4*>(xs + xs_index<KIND>(4 * g));
        float t = __fadd_rn(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y));
        t = __fadd_rn(t, __fmul_rn(a.z, b.z));
        t = __fadd_rn(t, __fmul_rn(a.w, b.w));
        gs[g] = t;
    }
    __syncwarp();
    float chain = 0.0f;
    if (lane == 0) {
#pragma unroll 8
        for (int g = 0; g < groups; ++g) chain = __fadd_rn(chain, gs[g]);
        for (int k = groups << 2; k < d; ++k) chain = __fadd_rn(chain, __fmul_rn(xs[xs_index<KIND>(k)], wrow[k]));
    }
    __syncwarp();
    return chain;   // valid in lane 0
}

// One warp: softmax over ne logits, K rounds of arg-max (value descending, index
// ascending, candidates must exceed -1e30), renormalised mixture weights -
// core/math_cpu.cpp:546-558 and core/moe_cpu.cpp:85-98,233-254 bit for bit except
// exp(), evaluated in double and rounded.  s_p / s_sel: ne floats of scratch.
__device__ __forceinline__ void route_finish_warp(const float* __restrict__ logits, const float* __restrict__ bias,
                                                  int ne, int K, float* s_p, float* s_sel, int* s_idx, float* s_w,
                                                  float* probs_out, int lane) {
    float mx = logits[0];
    for (int e = lane; e < ne; e += 32) mx = fmaxf(mx, logits[e]);
    mx = warp_max(mx);
    for (int e = lane; e < ne; e += 32) s_p[e] = (float)exp((double)__fsub_rn(logits[e], mx));
    __syncwarp();
    float inv = 0.0f;
    if (lane == 0) {
        float sum = 0.0f;
        for (int e = 0; e < ne; ++e) sum = __fadd_rn(sum, s_p[e]);
        inv = (sum > 1e-12f) ? __fdiv_rn(1.0f, sum) : 0.0f;
    }
    inv = __shfl_sync(0xffffffffu, inv, 0);
    for (int e = lane; e < ne; e += 32) {
        const float pr = __fmul_rn(s_p[e], inv);
        s_p[e] = pr;
        s_sel[e] = bias ? __fadd_rn(pr, bias[e]) : pr;
        if (probs_out) probs_out[e] = pr;
    }
    __syncwarp();
    for (int k = 0; k < K; ++k) {
        float bv = -1e30f;
        int bi = -1;
        for (int e = lane; e < ne; e += 32) {
            bool taken = false;
            for (int j = 0; j < k; ++j) taken |= (s_idx[j] == e);
            const float v = s_sel[e];
            if (!taken && v > bv) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        if (lane == 0) s_idx[k] = bi < 0 ? 0 : bi;
        __syncwarp();
    }
    if (lane == 0) {
        float sum_w = 0.0f;
        for (int k = 0; k < K; ++k) { s_w[k] = s_p[s_idx[k]]; sum_w = __fadd_rn(sum_w, s_w[k]); }
        if (sum_w > 1e-8f) {
            const float inv_w = __fdiv_rn(1.0f, sum_w);
            for (int k = 0; k < K; ++k) s_w[k] = __fmul_rn(s_w[k], inv_w);
        } else {
            const float uni = __fdiv_rn(1.0f, (float)K);
            for (int k = 0; k < K; ++k) s_w[k] = uni;
        }
    }
    __syncwarp();
}

constexpr int ROUTER_ROWS = SG_CONSUMERS;     // one expert per consumer warp per router tile

// ---- phase 1: router logits (exact order) and the shared expert's gate/up ----
// tiles [0, n_router): ROUTER_ROWS fp32 router rows; then shared tiles: R rows of
// sh_gate followed by the same R rows of sh_up.
template <int KIND, int MT>
__global__ void __launch_bounds__(SG_THREADS) moe_phase1_kernel(MoeFusedArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    Ring ring;
    ring.stages = smem;
    ring.stage_bytes = a.stage_bytes;
    ring.n_stages = a.n_stages;
    ring.status = a.status;
    float* xs = reinterpret_cast<float*>(smem + (size_t)a.n_stages * a.stage_bytes);
    const int xs_tok = xs_floats(a.d);
    float* nw_s = xs + (size_t)MT * xs_tok;
    float* gs = nw_s + a.d;                                         // [SG_CONSUMERS][d/4]
    ring.full = reinterpret_cast<uint64_t*>(gs + SG_CONSUMERS * (a.d >> 2));
    ring.empty = ring.full + SG_MAX_STAGES;
    double* red = reinterpret_cast<double*>(ring.empty + SG_MAX_STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_router = (a.ne + ROUTER_ROWS - 1) / ROUTER_ROWS;
    const int n_shared = a.SH > 0 ? (a.SH + a.rows_per_tile - 1) / a.rows_per_tile : 0;
    const int num_tiles = n_router + n_shared;
    const int first = blockIdx.x, step = gridDim.x;
    const int n_my = first < num_tiles ? (num_tiles - first + step - 1) / step : 0;
    const int64_t rb = row_bytes_of(KIND, a.d);
    ring.init();
    if (threadIdx.x == 0) pdl_launch_dependents();

    if (warp == SG_CONSUMERS) {
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < n_my; ++i) {
                if (!ring.acquire(i)) break;
                const int tile = first + i * step;
                if (tile < n_router) {
                    const int rows = min(ROUTER_ROWS, a.ne - tile * ROUTER_ROWS);
                    const uint32_t bytes = (uint32_t)rows * a.d * 4;
                    ring.expect(i, bytes);
                    ring.copy(i, 0, a.router_w + (int64_t)tile * ROUTER_ROWS * a.d, bytes);
                } else {
                    const int r0 = (tile - n_router) * a.rows_per_tile;
                    const int rows = min(a.rows_per_tile, a.SH - r0);
                    const uint32_t bytes = (uint32_t)(rows * rb);
                    ring.expect(i, 2 * bytes);
                    ring.copy(i, 0, a.sh_g + r0 * rb, bytes);
                    ring.copy(i, a.rows_per_tile * (int)rb, a.sh_u + r0 * rb, bytes);
                }
                issued = i + 1;
            }
            ring.drain(issued);
        }
        return;
    }
    for (int k = threadIdx.x; k < a.d; k += SG_CTHREADS) nw_s[k] = a.norm_w[k];
    pdl_wait();
    for (int m = 0; m < a.M; ++m)
        stage_x<KIND, true>(a.x + (int64_t)m * a.d, nw_s, xs + m * xs_tok, a.d, a.eps, red);
    consumer_sync();

    for (int i = 0; i < n_my; ++i) {
        if (!ring.wait_full(i)) break;
        const int tile = first + i * step;
        const uint8_t* ts = ring.stage(i);
        if (tile < n_router) {
            const int e = tile * ROUTER_ROWS + warp;
            if (e < a.ne) {
                const float* wrow = reinterpret_cast<const float*>(ts) + (int64_t)warp * a.d;
                for (int m = 0; m < a.M; ++m) {
                    const float lg = router_logit<KIND>(wrow, xs + m * xs_tok, gs + warp * (a.d >> 2), a.d, lane);
                    if (lane == 0) a.logits[(int64_t)m * a.ne + e] = lg;
                }
            }
        } else {
            const int r0 = (tile - n_router) * a.rows_per_tile;
            const int rows = min(a.rows_per_tile, a.SH - r0);
            for (int r = warp; r < rows; r += SG_CONSUMERS) {
                float g[MT], u[MT];
                row_dot_xs<KIND, MT>(ts + (int64_t)r * rb, xs, xs_tok, a.M, a.d, lane, g);
                row_dot_xs<KIND, MT>(ts + (int64_t)(a.rows_per_tile + r) * rb, xs, xs_tok, a.M, a.d, lane, u);
                if (lane < MT && lane < a.M) {
                    float gv = 0.0f, uv = 0.0f;
#pragma unroll
                    for (int m = 0; m < MT; ++m)
                        if (m == lane) { gv = g[m]; uv = u[m]; }
                    a.sh_act[(int64_t)lane * a.SH + r0 + r] = silu_acc(gv) * uv;
                }
            }
        }
        ring.release(i);
    }
}

// ---- phase 2: finish the routing, routed experts' gate/up -----------------------
// grid (ctas, M): blockIdx.y is the token.  The producer warp turns the logits into
// (idx, w) - every CTA computes the same values, CTA x == 0 publishes them - then
// streams tiles (k, row tile) of expert idx[k]: R gate rows followed by R up rows.
template <int KIND>
__global__ void __launch_bounds__(SG_THREADS) moe_phase2_kernel(MoeFusedArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    Ring ring;
    ring.stages = smem;
    ring.stage_bytes = a.stage_bytes;
    ring.n_stages = a.n_stages;
    ring.status = a.status;
    float* xs = reinterpret_cast<float*>(smem + (size_t)a.n_stages * a.stage_bytes);
    const int xs_tok = xs_floats(a.d);
    float* nw_s = xs + xs_tok;
    float* s_p = nw_s + a.d;          // [ne]
    float* s_sel = s_p + a.ne;        // [ne]
    float* s_w = s_sel + a.ne;        // [16]
    int* s_idx = reinterpret_cast<int*>(s_w + 16);   // [16]
    ring.full = reinterpret_cast<uint64_t*>(s_idx + 16);
    ring.empty = ring.full + SG_MAX_STAGES;
    double* red = reinterpret_cast<double*>(ring.empty + SG_MAX_STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.y;
    const int tiles_per_slot = (a.E + a.rows_per_tile - 1) / a.rows_per_tile;
    const int num_tiles = a.K * tiles_per_slot;
    const int first = blockIdx.x, step = gridDim.x;
    const int n_my = first < num_tiles ? (num_tiles - first + step - 1) / step : 0;
    const int64_t rb = row_bytes_of(KIND, a.d);
    ring.init();
    if (threadIdx.x == 0) pdl_launch_dependents();

    if (warp == SG_CONSUMERS) {
        pdl_wait();
        route_finish_warp(a.logits + (int64_t)m * a.ne, a.router_bias, a.ne, a.K, s_p, s_sel, s_idx, s_w,
                          (blockIdx.x == 0 && a.probs_out) ? a.probs_out + (int64_t)m * a.ne : nullptr, lane);
        if (blockIdx.x == 0 && lane < a.K) {
            a.idx[(int64_t)m * a.K + lane] = s_idx[lane];
            a.w[(int64_t)m * a.K + lane] = s_w[lane];
        }
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < n_my; ++i) {
                if (!ring.acquire(i)) break;
                const int tile = first + i * step;
                const int k = tile / tiles_per_slot, r0 = (tile % tiles_per_slot) * a.rows_per_tile;
                const int rows = min(a.rows_per_tile, a.E - r0);
                const int64_t row0 = (int64_t)s_idx[k] * a.E + r0;
                const uint32_t bytes = (uint32_t)(rows * rb);
                ring.expect(i, 2 * bytes);
                ring.copy(i, 0, a.gates + row0 * rb, bytes);
                ring.copy(i, a.rows_per_tile * (int)rb, a.ups + row0 * rb, bytes);
                issued = i + 1;
            }
            ring.drain(issued);
        }
        return;
    }
    for (int k = threadIdx.x; k < a.d; k += SG_CTHREADS) nw_s[k] = a.norm_w[k];
    pdl_wait();
    stage_x<KIND, true>(a.x + (int64_t)m * a.d, nw_s, xs, a.d, a.eps, red);
    consumer_sync();
    for (int i = 0; i < n_my; ++i) {
        if (!ring.wait_full(i)) break;
        const int tile = first + i * step;
        const int k = tile / tiles_per_slot, r0 = (tile % tiles_per_slot) * a.rows_per_tile;
        const int rows = min(a.rows_per_tile, a.E - r0);
        const uint8_t* ts = ring.stage(i);
        for (int r = warp; r < rows; r += SG_CONSUMERS) {
            float g[1], u[1];
            row_dot_xs<KIND, 1>(ts + (int64_t)r * rb, xs, xs_tok, 1, a.d, lane, g);
            row_dot_xs<KIND, 1>(ts + (int64_t)(a.rows_per_tile + r) * rb, xs, xs_tok, 1, a.d, lane, u);
            if (lane == 0) a.act[((int64_t)m * a.K + k) * a.E + r0 + r] = silu_acc(g[0]) * u[0];
        }
        ring.release(i);
    }
}

// ---- phase 3: down projections, weighted combine in k order, residual add --------
// grid (ctas, M).  A tile is R output rows: R rows of sh_down (K = SH) followed, for
// each k, by R rows of down[idx[k]] (K = E).
template <int KIND>
__global__ void __launch_bounds__(SG_THREADS) moe_phase3_kernel(MoeFusedArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    Ring ring;
    ring.stages = smem;
    ring.stage_bytes = a.stage_bytes;
    ring.n_stages = a.n_stages;
    ring.status = a.status;
    float* xs_sh = reinterpret_cast<float*>(smem + (size_t)a.n_stages * a.stage_bytes);   // shared act, unit-major
    const int sh_fl = xs_floats(a.SH), e_fl = xs_floats(a.E);
    float* xs_e = xs_sh + sh_fl;                                                            // [K] routed acts
    float* s_w = xs_e + (size_t)a.K * e_fl;       // [16]
    int* s_idx = reinterpret_cast<int*>(s_w + 16);
    ring.full = reinterpret_cast<uint64_t*>(s_idx + 16);
    ring.empty = ring.full + SG_MAX_STAGES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.y;
    const int num_tiles = (a.d + a.rows_per_tile - 1) / a.rows_per_tile;
    const int first = blockIdx.x, step = gridDim.x;
    const int n_my = first < num_tiles ? (num_tiles - first + step - 1) / step : 0;
    const int64_t rb_sh = a.SH > 0 ? row_bytes_of(KIND, a.SH) : 0, rb_e = row_bytes_of(KIND, a.E);
    const int sub_sh = a.rows_per_tile * (int)rb_sh, sub_e = a.rows_per_tile * (int)rb_e;
    ring.init();
    if (threadIdx.x == 0) pdl_launch_dependents();

    if (warp == SG_CONSUMERS) {
        pdl_wait();
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < n_my; ++i) {
                if (!ring.acquire(i)) break;
                const int r0 = (first + i * step) * a.rows_per_tile;
                const int rows = min(a.rows_per_tile, a.d - r0);
                ring.expect(i, (uint32_t)(rows * (rb_sh + a.K * rb_e)));
                if (a.SH > 0) ring.copy(i, 0, a.sh_d + r0 * rb_sh, (uint32_t)(rows * rb_sh));
                for (int k = 0; k < a.K; ++k) {
                    const int e = a.idx[(int64_t)m * a.K + k];
                    ring.copy(i, sub_sh + k * sub_e, a.downs + ((int64_t)e * a.d + r0) * rb_e, (uint32_t)(rows * rb_e));
                }
                issued = i + 1;
            }
            ring.drain(issued);
        }
        return;
    }
    pdl_wait();
    if (threadIdx.x < a.K) s_w[threadIdx.x] = a.w[(int64_t)m * a.K + threadIdx.x];
    for (int k = threadIdx.x; k < a.SH; k += SG_CTHREADS) xs_sh[xs_index<KIND>(k)] = a.sh_act[(int64_t)m * a.SH + k];
    for (int k = threadIdx.x; k < a.K * a.E; k += SG_CTHREADS) {
        const int slot = k / a.E, c = k - slot * a.E;
        xs_e[slot * e_fl + xs_index<KIND>(c)] = a.act[((int64_t)m * a.K + slot) * a.E + c];
    }
    consumer_sync();
    for (int i = 0; i < n_my; ++i) {
        const int r0 = (first + i * step) * a.rows_per_tile;
        const int rows = min(a.rows_per_tile, a.d - r0);
        if (!ring.wait_full(i)) break;
        const uint8_t* ts = ring.stage(i);
        for (int r = warp; r < rows; r += SG_CONSUMERS) {
            float* dst = a.resid + (int64_t)m * a.d + r0 + r;
            float pre = 0.0f;
            if (lane == 0) pre = *dst;
            float acc = 0.0f, t[1];
            if (a.SH > 0) {
                row_dot_xs<KIND, 1>(ts + (int64_t)r * rb_sh, xs_sh, sh_fl, 1, a.SH, lane, t);
                acc = t[0];
            }
            for (int k = 0; k < a.K; ++k) {
                row_dot_xs<KIND, 1>(ts + sub_sh + k * sub_e + (int64_t)r * rb_e, xs_e + k * e_fl, e_fl, 1, a.E, lane, t);
                acc = __fadd_rn(acc, __fmul_rn(s_w[k], t[0]));
            }
            if (lane == 0) *dst = pre + acc * a.res_mult;
        }
        ring.release(i);
    }
}

// ===========================================================================
// host side
// ===========================================================================
template <typename Kern, typename Args>
static int launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, const Args& a) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
    ++g_kernel_launches;
    return B200_OK;
}

template <typename Kern>
static int allow_smem(Kern kern) {
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET));
    return B200_OK;
}

// rows per tile: about `target` bytes, a multiple of what keeps tiles 16-byte aligned
static int pick_rows(int64_t bytes_per_row, int64_t align_row_bytes, int max_rows, int target = 8192) {
    int align_rows = 1;
    while ((align_rows * align_row_bytes) % 16 != 0 && align_rows < 16) align_rows *= 2;
    if ((align_rows * align_row_bytes) % 16 != 0) return -1;
    int R = (int)std::max<int64_t>(1, target / std::max<int64_t>(1, bytes_per_row));
    R = std::max(align_rows, R / align_rows * align_rows);
    R = std::min(R, std::max(align_rows, max_rows / align_rows * align_rows));
    return std::min(R, 64);
}

static int pick_stages(size_t stage_bytes, size_t other_bytes) {
    int s = SG_MAX_STAGES;
    while (s > 1 && s * stage_bytes + other_bytes > (size_t)SMEM_BUDGET) --s;
    return (s * stage_bytes + other_bytes <= (size_t)SMEM_BUDGET) ? s : 0;
}

template <int KIND, int MT, int PRO, int EPI>
static int launch_sg_inst(const SgArgs& a, int grid, size_t smem) {
    auto kern = stream_gemv_kernel<KIND, MT, PRO, EPI>;
    static bool configured = false;
    if (!configured) {
        int rc = allow_smem(kern);
        if (rc) return rc;
        configured = true;
    }
    return launch_pdl(kern, dim3(grid), dim3(SG_THREADS), smem, a);
}

static size_t sg_other_bytes(const SgArgs& a, int mt, int pro) {
    return (size_t)mt * xs_floats(a.K) * 4 + (pro == PRO_RMS ? (size_t)a.K * 4 : 0) + 2 * SG_MAX_STAGES * 8 + 64;
}

template <int KIND, int PRO, int EPI>
static int launch_sg_mt(SgArgs a, int grid) {
    const int mt = a.M == 1 ? 1 : a.M == 2 ? 2 : a.M <= 4 ? 4 : 8;
    const size_t other = sg_other_bytes(a, mt, PRO);
    a.n_stages = pick_stages(a.stage_bytes, other);
    if (a.n_stages < 2) return fail(B200_EUNSUPPORTED, "stream_gemv: K = %d does not fit the shared-memory staging", a.K);
    const size_t smem = (size_t)a.n_stages * a.stage_bytes + other;
    if (mt == 1) return launch_sg_inst<KIND, 1, PRO, EPI>(a, grid, smem);
    if (mt == 2) return launch_sg_inst<KIND, 2, PRO, EPI>(a, grid, smem);
    if (mt == 4) return launch_sg_inst<KIND, 4, PRO, EPI>(a, grid, smem);
    return launch_sg_inst<KIND, 8, PRO, EPI>(a, grid, smem);
}

// Fills the tiling fields and launches.  kind: template tag.
int stream_gemv(SgArgs a, int kind, int pro, int epi) {
    B200_REQUIRE(a.M >= 1 && a.M <= 8, "stream_gemv: 1..8 tokens per launch");
    B200_REQUIRE(a.K % 32 == 0 && (kind != 3 || a.K % 256 == 0), "stream_gemv: K not a multiple of the block size");
    a.row_bytes = row_bytes_of(kind, a.K);
    const int R = pick_rows(a.row_bytes, a.row_bytes, a.N);
    if (R < 1) return fail(B200_EUNSUPPORTED, "stream_gemv: row size %lld cannot be tiled to 16 bytes", (long long)a.row_bytes);
    a.rows_per_tile = R;
    a.num_tiles = ceil_div(a.N, R);
    a.stage_bytes = (int)((R * a.row_bytes + 127) / 128 * 128);
    a.status = stream_status_ptr();
    B200_REQUIRE(a.status, "stream_gemv: status word allocation failed");
    B200_REQUIRE((reinterpret_cast<uintptr_t>(a.w) & 15) == 0, "stream_gemv: weights must be 16-byte aligned");
    const int grid = std::min(a.num_tiles, 2 * num_sms());
#define SG_DISPATCH(KIND)                                                                                   \
    if (pro == PRO_RMS && epi == EPI_STORE) return launch_sg_mt<KIND, PRO_RMS, EPI_STORE>(a, grid);         \
    if (pro == PRO_RMS && epi == EPI_INPROJ) return launch_sg_mt<KIND, PRO_RMS, EPI_INPROJ>(a, grid);       \
    if (pro == PRO_NONE && epi == EPI_RESIDUAL) return launch_sg_mt<KIND, PRO_NONE, EPI_RESIDUAL>(a, grid); \
    if (pro == PRO_NONE && epi == EPI_STORE) return launch_sg_mt<KIND, PRO_NONE, EPI_STORE>(a, grid);       \
    return fail(B200_EINVAL, "stream_gemv: unsupported prologue/epilogue pair");
    switch (kind) {
        case 0: SG_DISPATCH(0)
        case 1: SG_DISPATCH(1)
        case 2: SG_DISPATCH(2)
        case 3: SG_DISPATCH(3)
        case KIND_F16: SG_DISPATCH(KIND_F16)
        default: SG_DISPATCH(KIND_F32)
    }
#undef SG_DISPATCH
}

int mamba_scan_norm_blocks(const MambaDims& p) { return ceil_div(p.n_heads * p.d_head, FS_WARPS); }

int mamba_scan_norm(const float* bc, const float* dt_raw, const float* gate, const float* dt_bias,
                    const float* a_log, const float* D, const float* norm_w, float* ssm_state, float* u_out,
                    double* partials, int batch, const MambaDims& p) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(mamba_scan_norm_blocks(p), batch);
    cfg.blockDim = dim3(FS_WARPS * 32);
    cfg.stream = stream();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200_CUDA(cudaLaunchKernelEx(&cfg, mamba_scan_norm_kernel, bc, dt_raw, gate, dt_bias, a_log, D, norm_w, ssm_state,
                                 u_out, partials, p));
    ++g_kernel_launches;
    return B200_OK;
}

// ---- MoE ----------------------------------------------------------------------
template <int KIND>
static int moe_fused_kind(MoeFusedArgs a) {
    const int64_t rb_d = row_bytes_of(KIND, a.d), rb_e = row_bytes_of(KIND, a.E);
    const int64_t rb_sh = a.SH > 0 ? row_bytes_of(KIND, a.SH) : 0;
    const int mt = a.M == 1 ? 1 : a.M == 2 ? 2 : a.M <= 4 ? 4 : 8;
    const size_t bars = 2 * SG_MAX_STAGES * 8 + 64;
    // ---- phase 1
    {
        MoeFusedArgs p1 = a;
        const int R = pick_rows(2 * rb_d, rb_d, std::max(a.SH, 1));
        if (R < 1) return fail(B200_EUNSUPPORTED, "moe_fused: row size cannot be tiled to 16 bytes");
        p1.rows_per_tile = R;
        const size_t stage = std::max<size_t>((size_t)ROUTER_ROWS * a.d * 4, (size_t)2 * R * rb_d);
        p1.stage_bytes = (int)((stage + 127) / 128 * 128);
        const size_t other = (size_t)mt * xs_floats(a.d) * 4 + (size_t)a.d * 4 + (size_t)SG_CONSUMERS * (a.d / 4) * 4 + bars;
        p1.n_stages = pick_stages(p1.stage_bytes, other);
        if (p1.n_stages < 2) return fail(B200_EUNSUPPORTED, "moe_fused: hidden size %d does not fit the shared-memory staging", a.d);
        const int tiles = ceil_div(a.ne, ROUTER_ROWS) + (a.SH > 0 ? ceil_div(a.SH, R) : 0);
        const size_t smem = (size_t)p1.n_stages * p1.stage_bytes + other;
        const int grid = std::min(tiles, 2 * num_sms());
        int rc;
#define P1(MT_)                                                        \
    {                                                                  \
        auto kern = moe_phase1_kernel<KIND, MT_>;                      \
        static bool cfgd = false;                                      \
        if (!cfgd) { rc = allow_smem(kern); if (rc) return rc; cfgd = true; } \
        rc = launch_pdl(kern, dim3(grid), dim3(SG_THREADS), smem, p1); \
    }
        if (mt == 1) P1(1) else if (mt == 2) P1(2) else if (mt == 4) P1(4) else P1(8)
#undef P1
        if (rc) return rc;
    }
    // ---- phase 2
    {
        MoeFusedArgs p2 = a;
        const int R = pick_rows(2 * rb_d, rb_d, a.E);
        p2.rows_per_tile = R;
        p2.stage_bytes = (int)(((size_t)2 * R * rb_d + 127) / 128 * 128);
        const size_t other = (size_t)xs_floats(a.d) * 4 + (size_t)a.d * 4 + (size_t)2 * a.ne * 4 + 128 + bars;
        p2.n_stages = pick_stages(p2.stage_bytes, other);
        if (p2.n_stages < 2) return fail(B200_EUNSUPPORTED, "moe_fused: hidden size %d does not fit the shared-memory staging", a.d);
        const int tiles = a.K * ceil_div(a.E, R);
        const int grid = std::max(1, std::min(tiles, (2 * num_sms()) / std::max(1, a.M)));
        auto kern = moe_phase2_kernel<KIND>;
        static bool cfgd = false;
        if (!cfgd) { int rc = allow_smem(kern); if (rc) return rc; cfgd = true; }
        int rc = launch_pdl(kern, dim3(grid, a.M), dim3(SG_THREADS), (size_t)p2.n_stages * p2.stage_bytes + other, p2);
        if (rc) return rc;
    }
    // ---- phase 3
    {
        MoeFusedArgs p3 = a;
        const int64_t per_row = rb_sh + (int64_t)a.K * rb_e;
        // every sub-tile (R rows of one matrix) must stay 16-byte aligned
        int R = pick_rows(per_row, rb_e, a.d);
        while (R >= 1 && R <= 64 && ((R * rb_sh) % 16 != 0 || (R * rb_e) % 16 != 0)) ++R;
        if (R < 1 || R > 64) return fail(B200_EUNSUPPORTED, "moe_fused: row size cannot be tiled to 16 bytes");
        p3.rows_per_tile = R;
        p3.stage_bytes = (int)(((size_t)R * per_row + 127) / 128 * 128);
        const size_t other = (size_t)(xs_floats(std::max(a.SH, 32)) + (size_t)a.K * xs_floats(a.E)) * 4 + 128 + bars;
        p3.n_stages = pick_stages(p3.stage_bytes, other);
        if (p3.n_stages < 2) return fail(B200_EUNSUPPORTED, "moe_fused: expert width does not fit the shared-memory staging");
        const int tiles = ceil_div(a.d, R);
        const int grid = std::max(1, std::min(tiles, (2 * num_sms()) / std::max(1, a.M)));
        auto kern = moe_phase3_kernel<KIND>;
        static bool cfgd = false;
        if (!cfgd) { int rc = allow_smem(kern); if (rc) return rc; cfgd = true; }
        int rc = launch_pdl(kern, dim3(grid, a.M), dim3(SG_THREADS), (size_t)p3.n_stages * p3.stage_bytes + other, p3);
        if (rc) return rc;
    }
    return B200_OK;
}

int moe_fused(MoeFusedArgs a, int kind) {
    B200_REQUIRE(a.M >= 1 && a.M <= 8, "moe_fused: 1..8 tokens per launch");
    B200_REQUIRE(a.K >= 1 && a.K <= 16 && a.ne >= a.K && a.ne <= 256, "moe_fused: K / ne out of range");
    B200_REQUIRE(a.d % 32 == 0 && a.E % 32 == 0 && a.SH % 32 == 0, "moe_fused: d, E, SH must be multiples of 32");
    if (kind == 3) B200_REQUIRE(a.d % 256 == 0 && a.E % 256 == 0 && a.SH % 256 == 0, "moe_fused: Q4_K needs multiples of 256");
    B200_REQUIRE((reinterpret_cast<uintptr_t>(a.router_w) & 15) == 0, "moe_fused: router_w must be 16-byte aligned");
    a.status = stream_status_ptr();
    B200_REQUIRE(a.status, "moe_fused: status word allocation failed");
    switch (kind) {
        case 0: return moe_fused_kind<0>(a);
        case 1: return moe_fused_kind<1>(a);
        case 2: return moe_fused_kind<2>(a);
        case 3: return moe_fused_kind<3>(a);
        case KIND_F16: return moe_fused_kind<KIND_F16>(a);
        default: return moe_fused_kind<KIND_F32>(a);
    }
}

}  // namespace b200
