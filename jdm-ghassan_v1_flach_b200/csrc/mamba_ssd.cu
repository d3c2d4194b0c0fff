// Chunked selective-state-space scan for Mamba-2 prefill (the "SSD" form).
//
// The recurrence of one head (core/mamba_cpu.cpp:120-170; state s [d_head, d_state]),
//     s_t = dA_t s_{t-1} + (dt_t B_t) x_t^T,      y_t = C_t . s_t + D x_t,
// is sequential in t.  Cut into chunks of SSD_Q steps it becomes dense algebra:
// with a_t = A dt_t (<= 0) and cum_t its running sum inside the chunk,
//     intra   Y[t] += sum_{s<=t} exp(cum_t - cum_s) (C_t . B_s) dt_s x_s
//     state   S_c   = sum_s exp(cum_last - cum_s) dt_s x_s B_s^T       (chunk's own contribution)
//     carry   S_prev(c+1) = exp(cum_last(c)) S_prev(c) + S_c              (sequential over chunks only)
//     inter   Y[t] += exp(cum_t) C_t . S_prev(c)
// so all T steps of all heads run in parallel except the short carry over chunks.
// B and C are shared by the heads (n_groups == 1), hence C_t . B_s is computed once per
// (sequence, chunk).  Everything is fp32; only the order of additions differs from the
// sequential scan (which the reference itself has no chunked form of: its
// mamba_chunk_size option is parsed and unused).
//
//   ssd_cb_kernel           G[b,c] = C B^T                         [Q, Q]
//   ssd_chunk_state_kernel  dt, cum per step; S_c per (b, c, h)   [d_head, d_state]
//   ssd_carry_kernel        S_c -> S_prev(c) in place, final state out
//   ssd_chunk_out_kernel    y = intra + inter + D x
#include "fused.cuh"

namespace b200 {

constexpr int SSD_Q = 128;                 // steps per chunk
constexpr int SSD_THREADS = 256;

__device__ __forceinline__ float softplus_dt(float u) { return (u > 20.0f) ? u : log1pf(expf(u)); }

// ---- G = C B^T per (sequence, chunk) ---------------------------------------------
// grid (chunks, B); thread (ty, tx) of a 16 x 16 block owns an 8 x 8 block of G.
__global__ void __launch_bounds__(SSD_THREADS)
ssd_cb_kernel(const float* __restrict__ bc, float* __restrict__ G, int T, MambaDims p) {
    extern __shared__ float sm[];
    const int N = p.d_state, ld = N + 1;
    float* sC = sm;                         // [Q][ld]
    float* sB = sm + SSD_Q * ld;            // [Q][ld]
    const int c = blockIdx.x, b = blockIdx.y;
    const int t0 = c * SSD_Q, nt = min(SSD_Q, T - t0);
    for (int e = threadIdx.x; e < SSD_Q * N; e += SSD_THREADS) {
        const int t = e / N, n = e - t * N;
        float bv = 0.0f, cv = 0.0f;
        if (t < nt) {
            const float* row = bc + ((int64_t)b * T + t0 + t) * p.conv_dim + p.d_inner;
            bv = row[n];
            cv = row[N + n];
        }
        sB[t * ld + n] = bv;
        sC[t * ld + n] = cv;
    }
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[8][8] = {};
    for (int n = 0; n < N; ++n) {
        float cv[8], bv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) cv[i] = sC[(ty * 8 + i) * ld + n];
#pragma unroll
        for (int j = 0; j < 8; ++j) bv[j] = sB[(tx * 8 + j) * ld + n];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] += cv[i] * bv[j];
    }
    float* g = G + ((int64_t)b * gridDim.x + c) * SSD_Q * SSD_Q;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) g[(ty * 8 + i) * SSD_Q + tx * 8 + j] = acc[i][j];
}

// ---- per (chunk, head, sequence): dt, cum, chunk state ----------------------------
// dtcum: [B, H, T, 2] (dt, cum).  chunk_state: [B, NC, H, P, N].  decay: [B, NC, H].
__global__ void __launch_bounds__(SSD_THREADS)
ssd_chunk_state_kernel(const float* __restrict__ proj, const float* __restrict__ bc, const float* __restrict__ dt_bias,
                       const float* __restrict__ a_log, float* __restrict__ dtcum, float* __restrict__ chunk_state,
                       float* __restrict__ decay, int T, int NC, MambaDims p) {
    extern __shared__ float sm[];
    const int N = p.d_state, P = p.d_head;
    float* sB = sm;                         // [Q][N]
    float* sX = sB + SSD_Q * N;             // [Q][P]   (already multiplied by w_s)
    float* sDt = sX + SSD_Q * P;            // [Q]
    float* sCum = sDt + SSD_Q;              // [Q]
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int t0 = c * SSD_Q, nt = min(SSD_Q, T - t0);
    const float A = -expf(a_log[h]);
    if (threadIdx.x < SSD_Q) {
        float dt = 0.0f;
        if (threadIdx.x < nt) {
            const float u = proj[((int64_t)b * T + t0 + threadIdx.x) * p.proj + p.proj - p.n_heads + h] + dt_bias[h];
            dt = softplus_dt(u);
        }
        sDt[threadIdx.x] = dt;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float run = 0.0f;
        for (int t = 0; t < SSD_Q; ++t) {
            run += __fmul_rn(A, sDt[t]);
            sCum[t] = run;
        }
    }
    __syncthreads();
    const float cum_last = sCum[SSD_Q - 1];
    if (threadIdx.x < nt) {
        float* o = dtcum + (((int64_t)b * p.n_heads + h) * T + t0 + threadIdx.x) * 2;
        o[0] = sDt[threadIdx.x];
        o[1] = sCum[threadIdx.x];
    }
    if (threadIdx.x == 0) decay[((int64_t)b * NC + c) * p.n_heads + h] = expf(cum_last);
    for (int e = threadIdx.x; e < SSD_Q * N; e += SSD_THREADS) {
        const int t = e / N, n = e - t * N;
        sB[e] = t < nt ? bc[((int64_t)b * T + t0 + t) * p.conv_dim + p.d_inner + n] : 0.0f;
    }
    for (int e = threadIdx.x; e < SSD_Q * P; e += SSD_THREADS) {
        const int t = e / P, i = e - t * P;
        const float w = expf(cum_last - sCum[t]) * sDt[t];
        sX[e] = t < nt ? w * bc[((int64_t)b * T + t0 + t) * p.conv_dim + h * P + i] : 0.0f;
    }
    __syncthreads();
    // thread -> 8 rows (p) x 4 columns (n) of the state
    const int pgroups = P >> 3, ngroups = N >> 2;
    float* out = chunk_state + (((int64_t)b * NC + c) * p.n_heads + h) * P * N;
    for (int g = threadIdx.x; g < pgroups * ngroups; g += SSD_THREADS) {
        const int pg = g / ngroups, ng = g - pg * ngroups;
        float acc[8][4] = {};
        for (int s = 0; s < SSD_Q; ++s) {
            const float4 bv = *reinterpret_cast<const float4*>(sB + s * N + ng * 4);
            const float4 x0 = *reinterpret_cast<const float4*>(sX + s * P + pg * 8);
            const float4 x1 = *reinterpret_cast<const float4*>(sX + s * P + pg * 8 + 4);
            const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                acc[i][0] += xv[i] * bv.x;
                acc[i][1] += xv[i] * bv.y;
                acc[i][2] += xv[i] * bv.z;
                acc[i][3] += xv[i] * bv.w;
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(out + (pg * 8 + i) * N + ng * 4) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    }
}

// ---- carry over chunks: chunk_state[c] becomes the state BEFORE chunk c ------------
// one thread per state element of (b, h); sequential over the chunks.
__global__ void __launch_bounds__(256)
ssd_carry_kernel(float* __restrict__ chunk_state, const float* __restrict__ decay, float* __restrict__ state, int B,
                 int NC, MambaDims p) {
    const int64_t per = (int64_t)p.d_head * p.d_state;
    const int64_t total = (int64_t)B * p.n_heads * per;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t bh = i / per, e = i - bh * per;
        const int b = (int)(bh / p.n_heads), h = (int)(bh - (int64_t)b * p.n_heads);
        float s = state[i];
        for (int c = 0; c < NC; ++c) {
            float* cs = chunk_state + (((int64_t)b * NC + c) * p.n_heads + h) * per + e;
            const float own = *cs;
            *cs = s;
            s = decay[((int64_t)b * NC + c) * p.n_heads + h] * s + own;
        }
        state[i] = s;
    }
}

// ---- per (chunk, head, sequence): outputs ------------------------------------------
// thread -> 4 steps (t) x 8 channels (p).  Shared memory is used twice: first C and the
// transposed incoming state (inter-chunk term), then the masked, decayed G and x.
__global__ void __launch_bounds__(SSD_THREADS)
ssd_chunk_out_kernel(const float* __restrict__ bc, const float* __restrict__ G, const float* __restrict__ dtcum,
                     const float* __restrict__ chunk_state, const float* __restrict__ Dv, float* __restrict__ y, int T,
                     int NC, MambaDims p) {
    extern __shared__ float sm[];
    const int N = p.d_state, P = p.d_head;
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int t0 = c * SSD_Q, nt = min(SSD_Q, T - t0);
    float* sDt = sm;                        // [Q]
    float* sCum = sDt + SSD_Q;              // [Q]
    float* buf = sCum + SSD_Q;
    if (threadIdx.x < SSD_Q) {
        float dt = 0.0f, cum = 0.0f;
        if (threadIdx.x < nt) {
            const float* o = dtcum + (((int64_t)b * p.n_heads + h) * T + t0 + threadIdx.x) * 2;
            dt = o[0];
            cum = o[1];
        }
        sDt[threadIdx.x] = dt;
        sCum[threadIdx.x] = cum;
    }
    const int tgroups = SSD_Q >> 2, pgroups = P >> 3;
    const int items = tgroups * pgroups;    // <= SSD_THREADS for d_head <= 64; looped otherwise
    // phase 1: inter-chunk term
    {
        float* sC = buf;                    // [Q][N]
        float* sS = buf + SSD_Q * N;        // [N][P + 4]  (transposed state)
        const int lds = P + 4;
        for (int e = threadIdx.x; e < SSD_Q * N; e += SSD_THREADS) {
            const int t = e / N, n = e - t * N;
            sC[e] = t < nt ? bc[((int64_t)b * T + t0 + t) * p.conv_dim + p.d_inner + N + n] : 0.0f;
        }
        const float* sp = chunk_state + (((int64_t)b * NC + c) * p.n_heads + h) * P * N;
        for (int e = threadIdx.x; e < P * N; e += SSD_THREADS) {
            const int i = e / N, n = e - i * N;
            sS[n * lds + i] = sp[e];
        }
    }
    __syncthreads();
    for (int it = threadIdx.x; it < items; it += SSD_THREADS) {
        const int tg = it / pgroups, pg = it - tg * pgroups;
        float acc[4][8] = {};
        {
            const float* sC = buf;
            const float* sS = buf + SSD_Q * N;
            const int lds = P + 4;
            for (int n = 0; n < N; ++n) {
                const float4 s0 = *reinterpret_cast<const float4*>(sS + n * lds + pg * 8);
                const float4 s1 = *reinterpret_cast<const float4*>(sS + n * lds + pg * 8 + 4);
                const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float cv = sC[(tg * 4 + i) * N + n];
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[i][j] += cv * sv[j];
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float e = expf(sCum[tg * 4 + i]);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] *= e;
            }
        }
        __syncthreads();                     // (items <= SSD_THREADS: every thread passes here exactly once)
        // phase 2: intra-chunk term with M[t][s] = G[t][s] exp(cum_t - cum_s) dt_s for s <= t
        float* sM = buf;                    // [Q][Q + 1]
        float* sX = buf + SSD_Q * (SSD_Q + 1);   // [Q][P]
        {
            const float* g = G + ((int64_t)b * NC + c) * SSD_Q * SSD_Q;
            for (int e = threadIdx.x; e < SSD_Q * SSD_Q; e += SSD_THREADS) {
                const int t = e / SSD_Q, s = e - t * SSD_Q;
                sM[t * (SSD_Q + 1) + s] = (s <= t && t < nt) ? g[e] * expf(sCum[t] - sCum[s]) * sDt[s] : 0.0f;
            }
            for (int e = threadIdx.x; e < SSD_Q * P; e += SSD_THREADS) {
                const int t = e / P, i = e - t * P;
                sX[e] = t < nt ? bc[((int64_t)b * T + t0 + t) * p.conv_dim + h * P + i] : 0.0f;
            }
        }
        __syncthreads();
        const int s_end = min(nt, tg * 4 + 4);
        for (int s = 0; s < s_end; ++s) {
            const float4 x0 = *reinterpret_cast<const float4*>(sX + s * P + pg * 8);
            const float4 x1 = *reinterpret_cast<const float4*>(sX + s * P + pg * 8 + 4);
            const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float m = sM[(tg * 4 + i) * (SSD_Q + 1) + s];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] += m * xv[j];
            }
        }
        const float dskip = Dv[h];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int t = tg * 4 + i;
            if (t < nt) {
                float* o = y + ((int64_t)b * T + t0 + t) * p.d_inner + h * P + pg * 8;
                const float* xr = sX + t * P + pg * 8;
                *reinterpret_cast<float4*>(o) = make_float4(acc[i][0] + dskip * xr[0], acc[i][1] + dskip * xr[1],
                                                            acc[i][2] + dskip * xr[2], acc[i][3] + dskip * xr[3]);
                *reinterpret_cast<float4*>(o + 4) = make_float4(acc[i][4] + dskip * xr[4], acc[i][5] + dskip * xr[5],
                                                                acc[i][6] + dskip * xr[6], acc[i][7] + dskip * xr[7]);
            }
        }
    }
}

// The chunked scan over proj / bc (as produced by the projection and the convolution):
// y [B*T, d_inner], state [B, H, P, N] updated in place.  Returns B200_EUNSUPPORTED for
// shapes outside its tiling (the caller then runs the sequential scan).
int mamba_ssd_scan(const float* proj, const float* bc, const float* dt_bias, const float* a_log, const float* D,
                   float* state, float* y, int B, int T, const MambaDims& p) {
    const int N = p.d_state, P = p.d_head;
    if (N % 4 != 0 || P % 8 != 0 || (SSD_Q / 4) * (P / 8) != SSD_THREADS || N > 128 || (p.d_inner & 3) != 0)
        return fail(B200_EUNSUPPORTED, "mamba_ssd_scan: d_head %d / d_state %d outside the chunked kernels' tiling", P, N);
    const int NC = ceil_div(T, SSD_Q);
    const size_t g_f = (size_t)B * NC * SSD_Q * SSD_Q, dc_f = (size_t)B * p.n_heads * T * 2,
                 cs_f = (size_t)B * NC * p.n_heads * P * N, de_f = (size_t)B * NC * p.n_heads;
    void* wsp;
    int rc = workspace(WS_ATTN).ensure((g_f + dc_f + cs_f + de_f) * sizeof(float) + 1024, &wsp);
    if (rc) return rc;
    float* G = static_cast<float*>(wsp);
    float* dtcum = G + g_f;
    float* cstate = dtcum + ((dc_f + 3) & ~(size_t)3);
    float* decay = cstate + cs_f;
    const size_t smem_cb = (size_t)2 * SSD_Q * (N + 1) * 4;
    const size_t smem_st = (size_t)(SSD_Q * N + SSD_Q * P + 2 * SSD_Q) * 4;
    const size_t smem_out = (size_t)(2 * SSD_Q + std::max(SSD_Q * N + N * (P + 4), SSD_Q * (SSD_Q + 1) + SSD_Q * P)) * 4;
    static bool configured = false;
    if (!configured) {
        B200_CUDA(cudaFuncSetAttribute(ssd_cb_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        B200_CUDA(cudaFuncSetAttribute(ssd_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        B200_CUDA(cudaFuncSetAttribute(ssd_chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        configured = true;
    }
    B200_REQUIRE(smem_cb <= 160 * 1024 && smem_st <= 160 * 1024 && smem_out <= 160 * 1024, "mamba_ssd_scan: shared memory");
    B200_REQUIRE(NC <= 65535 * 32 && B <= 65535 && p.n_heads <= 65535, "mamba_ssd_scan: grid too large");
    ssd_cb_kernel<<<dim3(NC, B), SSD_THREADS, smem_cb, stream()>>>(bc, G, T, p);
    B200_LAUNCH_CHECK("ssd_cb_kernel");
    ssd_chunk_state_kernel<<<dim3(NC, p.n_heads, B), SSD_THREADS, smem_st, stream()>>>(proj, bc, dt_bias, a_log, dtcum, cstate,
                                                                                      decay, T, NC, p);
    B200_LAUNCH_CHECK("ssd_chunk_state_kernel");
    const int64_t elems = (int64_t)B * p.n_heads * P * N;
    ssd_carry_kernel<<<(unsigned)std::min<int64_t>(ceil_div64(elems, 256), (int64_t)num_sms() * 16), 256, 0, stream()>>>(
        cstate, decay, state, B, NC, p);
    B200_LAUNCH_CHECK("ssd_carry_kernel");
    ssd_chunk_out_kernel<<<dim3(NC, p.n_heads, B), SSD_THREADS, smem_out, stream()>>>(bc, G, dtcum, cstate, D, y, T, NC, p);
    B200_LAUNCH_CHECK("ssd_chunk_out_kernel");
    return B200_OK;
}

}  // namespace b200
