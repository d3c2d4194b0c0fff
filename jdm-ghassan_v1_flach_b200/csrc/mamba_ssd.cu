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
// (sequence, chunk).  dt, the running sums, the exponentials, the carry and all
// accumulation are fp32.  With fp32 weights (`precise`) the two per-head products run as
// split-TF32 (3 MMAs per product, fp32-level accuracy: only the order of additions differs
// from the sequential scan); with fp16 / packed weights - where the projections around the
// scan already round their activations to fp16 - their operands are rounded to TF32 once.
// (The reference has no chunked form to compare with: its mamba_chunk_size option is
// parsed and unused, and its scan is the sequential one.)
//
//   ssd_cb_kernel           G[b,c] = C B^T                         [Q, Q]
//   ssd_chunk_state_kernel  dt, cum per step; S_c per (b, c, h)   [d_head, d_state]
//   ssd_carry_kernel        S_c -> S_prev(c) in place, final state out
//   ssd_chunk_out_kernel    y = intra + inter + D x
#include "fused.cuh"

namespace b200 {

constexpr int SSD_THREADS = 256;            // (SSD_Q, the steps per chunk, is in fused.cuh)

// Where chunk c of sequence b lives.  Rectangular batches [B, T]: chunk c covers steps
// c SSD_Q .. of every sequence.  Packed sequences of different lengths (tab != nullptr,
// grid z = 1): chunk c is entry c of the table (first row, steps), which never crosses a
// sequence boundary; per-chunk arrays are indexed by c and dtcum is [H, NT, 2].
struct SsdChunk {
    int64_t row0;      // first row of the chunk in proj / bc / y
    int64_t ci;        // index into the per-chunk arrays (G, chunk_state, decay)
    int64_t dt0;       // index of the chunk's first (dt, cum) pair for head h
    int nt;            // steps in the chunk
};
__device__ __forceinline__ SsdChunk ssd_chunk(const int2* __restrict__ tab, int64_t NT, int c, int b, int h, int T, int NC,
                                              int H) {
    SsdChunk k;
    if (tab) {
        const int2 e = tab[c];
        k.row0 = e.x;
        k.nt = e.y;
        k.ci = c;
        k.dt0 = (int64_t)h * NT + e.x;
    } else {
        const int t0 = c * SSD_Q;
        k.row0 = (int64_t)b * T + t0;
        k.nt = min(SSD_Q, T - t0);
        k.ci = (int64_t)b * NC + c;
        k.dt0 = ((int64_t)b * H + h) * T + t0;
    }
    return k;
}

__device__ __forceinline__ float softplus_dt(float u) { return (u > 20.0f) ? u : log1pf(expf(u)); }

// ---- G = C B^T per (sequence, chunk) ---------------------------------------------
// Only s <= t is ever used, so of the four 64 x 64 quadrants of G the upper right one is
// skipped: grid (3 * chunks, B), quadrant (0,0), (1,0) or (1,1) per block; thread
// (ty, tx) of a 16 x 16 block owns a 4 x 4 block of its quadrant.  fp32 throughout.
__global__ void __launch_bounds__(SSD_THREADS)
ssd_cb_kernel(const float* __restrict__ bc, float* __restrict__ G, int T, MambaDims p, const int2* __restrict__ tab) {
    extern __shared__ float sm[];
    constexpr int H = SSD_Q / 2;
    const int N = p.d_state, ld = N + 1;
    float* sC = sm;                         // [H][ld]
    float* sB = sm + H * ld;                // [H][ld]
    const int c = blockIdx.x / 3, quad = blockIdx.x - 3 * c, b = blockIdx.y;
    const int NC = gridDim.x / 3;
    const int ti = quad == 0 ? 0 : H, si = quad == 2 ? H : 0;        // first row (t) and column (s)
    const SsdChunk ck = ssd_chunk(tab, 0, c, b, 0, T, NC, 1);
    const int nt = ck.nt;
    for (int e = threadIdx.x; e < H * N; e += SSD_THREADS) {
        const int r = e / N, n = e - r * N;
        float bv = 0.0f, cv = 0.0f;
        if (si + r < nt) bv = bc[(ck.row0 + si + r) * p.conv_dim + p.d_inner + n];
        if (ti + r < nt) cv = bc[(ck.row0 + ti + r) * p.conv_dim + p.d_inner + N + n];
        sB[r * ld + n] = bv;
        sC[r * ld + n] = cv;
    }
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[4][4] = {};
    for (int n = 0; n < N; ++n) {
        float cv[4], bv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) cv[i] = sC[(ty * 4 + i) * ld + n];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = sB[(tx * 4 + j) * ld + n];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] += cv[i] * bv[j];
    }
    float* g = G + (ck.ci) * SSD_Q * SSD_Q;
#pragma unroll
    for (int i = 0; i < 4; ++i)
        *reinterpret_cast<float4*>(g + (ti + ty * 4 + i) * SSD_Q + si + tx * 4) =
            make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
}

// ---- tensor-core pieces ---------------------------------------------------------------
// The two dense products per (chunk, head) run on mma.sync.m16n8k8 with TF32 operands
// (fp32 range, 11 significant bits) and fp32 accumulation; shared memory holds the fp32
// operands and they are rounded (or split, see Tf32Val) as fragments are loaded.  Leading
// dimensions are padded so that every fragment load of a warp touches 32 different banks.
__device__ __forceinline__ float tf32_round(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const float (&a)[4], float b0, float b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(__float_as_uint(a[0])), "r"(__float_as_uint(a[1])), "r"(__float_as_uint(a[2])),
          "r"(__float_as_uint(a[3])), "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

// One operand element as the tensor core sees it.  X3 = false: the value rounded to
// TF32.  X3 = true: the value split into a TF32 head and a TF32 tail, and a product is
// three MMAs (tail x head, head x tail, head x head), which restores fp32-level accuracy
// (the dropped tail x tail term is below 2^-22 relative).
template <bool X3>
struct Tf32Val {
    float hi, lo;
    __device__ __forceinline__ explicit Tf32Val(float v) : hi(tf32_round(v)), lo(X3 ? tf32_round(v - hi) : 0.0f) {}
    __device__ __forceinline__ Tf32Val() : hi(0.0f), lo(0.0f) {}
};
template <bool X3>
__device__ __forceinline__ void mma_x(float (&c)[4], const Tf32Val<X3> (&a)[4], const Tf32Val<X3>& b0, const Tf32Val<X3>& b1) {
    const float ah[4] = {a[0].hi, a[1].hi, a[2].hi, a[3].hi};
    if (X3) {
        const float al[4] = {a[0].lo, a[1].lo, a[2].lo, a[3].lo};
        mma_tf32(c, al, b0.hi, b1.hi);
        mma_tf32(c, ah, b0.lo, b1.lo);
    }
    mma_tf32(c, ah, b0.hi, b1.hi);
}

constexpr int SSD_P = 64;                  // d_head of the tensor-core kernels
constexpr int SSD_LDX = SSD_P + 8;         // x tile [Q][P + 8]

// ---- per (chunk, head, sequence): dt, cum, chunk state ----------------------------
// dtcum: [B, H, T, 2] (dt, cum).  chunk_state: [B, NC, H, P, N].  decay: [B, NC, H].
// S[p][n] = sum_s (w_s x[s][p]) B[s][n]: warp w owns rows 16 (w & 3) .. +16 and the
// (w >> 2)-th half of the columns.
template <bool X3>
__global__ void __launch_bounds__(SSD_THREADS, 2)
ssd_chunk_state_kernel(const float* __restrict__ proj, const float* __restrict__ bc, const float* __restrict__ dt_bias,
                       const float* __restrict__ a_log, float* __restrict__ dtcum, float* __restrict__ chunk_state,
                       float* __restrict__ decay, int T, int NC, MambaDims p, const int2* __restrict__ tab, int64_t NT) {
    extern __shared__ float sm[];
    constexpr int P = SSD_P;
    const int N = p.d_state, ldb = N + 8;
    float* sB = sm;                         // [Q][N + 8]
    float* sX = sB + SSD_Q * ldb;           // [Q][P + 8]   (already multiplied by w_s)
    float* sDt = sX + SSD_Q * SSD_LDX;      // [Q]
    float* sCum = sDt + SSD_Q;              // [Q]
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const SsdChunk ck = ssd_chunk(tab, NT, c, b, h, T, NC, p.n_heads);
    const int nt = ck.nt;
    const float A = -expf(a_log[h]);
    if (threadIdx.x < SSD_Q) {
        float dt = 0.0f;
        if (threadIdx.x < nt) {
            const float u = proj[(ck.row0 + threadIdx.x) * p.proj + p.proj - p.n_heads + h] + dt_bias[h];
            dt = softplus_dt(u);
        }
        sDt[threadIdx.x] = dt;
    }
    __syncthreads();
    if (threadIdx.x < 32) {                 // running sum of A dt over the chunk: 4 steps per lane
        const int l = threadIdx.x;
        float v[4], run = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            run += __fmul_rn(A, sDt[l * 4 + i]);
            v[i] = run;
        }
        float incl = run;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, incl, o);
            if (l >= o) incl += up;
        }
        const float before = incl - run;
#pragma unroll
        for (int i = 0; i < 4; ++i) sCum[l * 4 + i] = before + v[i];
    }
    __syncthreads();
    const float cum_last = sCum[SSD_Q - 1];
    if (threadIdx.x < nt) {
        float* o = dtcum + (ck.dt0 + threadIdx.x) * 2;
        o[0] = sDt[threadIdx.x];
        o[1] = sCum[threadIdx.x];
    }
    if (threadIdx.x == 0) decay[(ck.ci) * p.n_heads + h] = expf(cum_last);
    const int n4 = N >> 2;
    for (int e = threadIdx.x; e < SSD_Q * n4; e += SSD_THREADS) {
        const int t = e / n4, n = (e - t * n4) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < nt) v = *reinterpret_cast<const float4*>(bc + (ck.row0 + t) * p.conv_dim + p.d_inner + n);
        *reinterpret_cast<float4*>(sB + t * ldb + n) = v;
    }
    for (int e = threadIdx.x; e < SSD_Q * (P / 4); e += SSD_THREADS) {
        const int t = e / (P / 4), i = (e - t * (P / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < nt) {
            const float w = expf(cum_last - sCum[t]) * sDt[t];
            v = *reinterpret_cast<const float4*>(bc + (ck.row0 + t) * p.conv_dim + h * P + i);
            v = make_float4(w * v.x, w * v.y, w * v.z, w * v.w);
        }
        *reinterpret_cast<float4*>(sX + t * SSD_LDX + i) = v;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int mt = warp & 3, nh = warp >> 2;
    const int nth = N >> 4;                 // column tiles (of 8) per half, <= 8
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
    const int ksteps = (nt + 7) >> 3;
    for (int ks = 0; ks < ksteps; ++ks) {
        const float* xa = sX + (ks * 8 + t4) * SSD_LDX + mt * 16 + g;
        const Tf32Val<X3> a[4] = {Tf32Val<X3>(xa[0]), Tf32Val<X3>(xa[8]), Tf32Val<X3>(xa[4 * SSD_LDX]),
                                  Tf32Val<X3>(xa[4 * SSD_LDX + 8])};
        const float* bb = sB + (ks * 8 + t4) * ldb + nh * nth * 8 + g;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (j < nth) mma_x<X3>(acc[j], a, Tf32Val<X3>(bb[j * 8]), Tf32Val<X3>(bb[j * 8 + 4 * ldb]));
    }
    float* out = chunk_state + ((ck.ci) * p.n_heads + h) * P * N;
#pragma unroll
    for (int j = 0; j < 8; ++j)
        if (j < nth) {
            const int n = (nh * nth + j) * 8 + 2 * t4;
            *reinterpret_cast<float2*>(out + (mt * 16 + g) * N + n) = make_float2(acc[j][0], acc[j][1]);
            *reinterpret_cast<float2*>(out + (mt * 16 + g + 8) * N + n) = make_float2(acc[j][2], acc[j][3]);
        }
}

// ---- carry over chunks: chunk_state[c] becomes the state BEFORE chunk c ------------
// one thread per state element of (b, h): grid (d_head d_state / 256, heads, sequences), so no
// index is divided; sequential over the chunks, eight chunks' loads in flight at a time.
__global__ void __launch_bounds__(256)
ssd_carry_kernel(float* __restrict__ chunk_state, const float* __restrict__ decay, float* __restrict__ state, int B,
                 int NC, MambaDims p, const int32_t* __restrict__ seq_chunk0) {
    const int per = p.d_head * p.d_state;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per) return;
    const int h = blockIdx.y, b = blockIdx.z;
    const int64_t cstride = (int64_t)p.n_heads * per;
    const int64_t i = ((int64_t)b * p.n_heads + h) * per + e;
    // the sequence's chunks are consecutive entries of the per-chunk arrays
    const int64_t c_first = seq_chunk0 ? seq_chunk0[b] : (int64_t)b * NC;
    const int nc = seq_chunk0 ? seq_chunk0[b + 1] - seq_chunk0[b] : NC;
    float* cs = chunk_state + (c_first * p.n_heads + h) * per + e;
    const float* dc = decay + c_first * p.n_heads + h;
    float s = state[i];
    for (int c0 = 0; c0 < nc; c0 += 8) {
        float own[8], de[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (c0 + j < nc) {
                own[j] = __ldcs(cs + (c0 + j) * cstride);
                de[j] = dc[(int64_t)(c0 + j) * p.n_heads];
            }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (c0 + j < nc) {
                cs[(c0 + j) * cstride] = s;
                s = de[j] * s + own[j];
            }
    }
    state[i] = s;
}

// ---- per (chunk, head, sequence): outputs ------------------------------------------
// y[t][p] = sum_n (e^{cum_t} C[t][n]) S_prev[p][n] + sum_{s<=t} M[t][s] x[s][p] + D x[t][p],
// M[t][s] = G[t][s] e^{cum_t - cum_s} dt_s.  Both sums are TF32 tensor-core products
// into the same accumulators; shared memory holds first (C, S_prev), then (M, x).
// Warp w owns 32 channels (half w >> 2) of the row tiles w & 3 and 7 - (w & 3): the
// causal product skips the step tiles above the diagonal, and this pairing gives
// every warp the same number of them.
template <bool X3>
__global__ void __launch_bounds__(SSD_THREADS, 2)
ssd_chunk_out_kernel(const float* __restrict__ bc, const float* __restrict__ G, const float* __restrict__ dtcum,
                     const float* __restrict__ chunk_state, const float* __restrict__ Dv, float* __restrict__ y, int T,
                     int NC, MambaDims p, const int2* __restrict__ tab, int64_t NT) {
    extern __shared__ float sm[];
    constexpr int P = SSD_P, LDM = SSD_Q + 4;
    const int N = p.d_state, ldc = N + 4;
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const SsdChunk ck = ssd_chunk(tab, NT, c, b, h, T, NC, p.n_heads);
    const int nt = ck.nt;
    float* sDt = sm;                        // [Q]
    float* sCum = sDt + SSD_Q;              // [Q]
    float* buf = sCum + SSD_Q;
    if (threadIdx.x < SSD_Q) {
        float dt = 0.0f, cum = 0.0f;
        if (threadIdx.x < nt) {
            const float2 o = *reinterpret_cast<const float2*>(dtcum + (ck.dt0 + threadIdx.x) * 2);
            dt = o.x;
            cum = o.y;
        }
        sDt[threadIdx.x] = dt;
        sCum[threadIdx.x] = cum;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int ph = warp >> 2;
    const int mts[2] = {warp & 3, 7 - (warp & 3)};
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;
    // phase 1: inter-chunk term
    {
        float* sC = buf;                    // [Q][N + 4], rows scaled by e^{cum_t}
        float* sS = buf + SSD_Q * ldc;      // [P][N + 4]
        const int n4 = N >> 2;
        for (int e = threadIdx.x; e < SSD_Q * n4; e += SSD_THREADS) {
            const int t = e / n4, n = (e - t * n4) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < nt) {
                const float w = expf(sCum[t]);
                v = *reinterpret_cast<const float4*>(bc + (ck.row0 + t) * p.conv_dim + p.d_inner + N + n);
                v = make_float4(w * v.x, w * v.y, w * v.z, w * v.w);
            }
            *reinterpret_cast<float4*>(sC + t * ldc + n) = v;
        }
        const float* sp = chunk_state + ((ck.ci) * p.n_heads + h) * P * N;
        for (int e = threadIdx.x; e < P * n4; e += SSD_THREADS) {
            const int i = e / n4, n = (e - i * n4) * 4;
            const float4 v = __ldcs(reinterpret_cast<const float4*>(sp + i * N + n));
            *reinterpret_cast<float4*>(sS + i * ldc + n) = v;
        }
        __syncthreads();
        for (int ks = 0; ks < (N >> 3); ++ks) {
            Tf32Val<X3> a[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float* ca = sC + (mts[i] * 16 + g) * ldc + ks * 8 + t4;
                a[i][0] = Tf32Val<X3>(ca[0]);
                a[i][1] = Tf32Val<X3>(ca[8 * ldc]);
                a[i][2] = Tf32Val<X3>(ca[4]);
                a[i][3] = Tf32Val<X3>(ca[8 * ldc + 4]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float* sb = sS + (ph * 32 + j * 8 + g) * ldc + ks * 8 + t4;
                const Tf32Val<X3> b0(sb[0]), b1(sb[4]);
                mma_x<X3>(acc[0][j], a[0], b0, b1);
                mma_x<X3>(acc[1][j], a[1], b0, b1);
            }
        }
    }
    __syncthreads();
    // phase 2: intra-chunk term
    {
        float* sM = buf;                    // [Q][Q + 4]
        float* sX = buf + SSD_Q * LDM;      // [Q][P + 8]
        const float* gm = G + (ck.ci) * SSD_Q * SSD_Q;
        for (int e = threadIdx.x; e < SSD_Q * (SSD_Q / 4); e += SSD_THREADS) {
            const int t = e / (SSD_Q / 4), s = (e - t * (SSD_Q / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s <= t && t < nt) {
                const float4 gv = *reinterpret_cast<const float4*>(gm + t * SSD_Q + s);
                const float ct = sCum[t];
                v.x = gv.x * expf(ct - sCum[s]) * sDt[s];
                if (s + 1 <= t) v.y = gv.y * expf(ct - sCum[s + 1]) * sDt[s + 1];
                if (s + 2 <= t) v.z = gv.z * expf(ct - sCum[s + 2]) * sDt[s + 2];
                if (s + 3 <= t) v.w = gv.w * expf(ct - sCum[s + 3]) * sDt[s + 3];
            }
            *reinterpret_cast<float4*>(sM + t * LDM + s) = v;
        }
        for (int e = threadIdx.x; e < SSD_Q * (P / 4); e += SSD_THREADS) {
            const int t = e / (P / 4), i = (e - t * (P / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < nt) v = *reinterpret_cast<const float4*>(bc + (ck.row0 + t) * p.conv_dim + h * P + i);
            *reinterpret_cast<float4*>(sX + t * SSD_LDX + i) = v;
        }
        __syncthreads();
        const int kmax = (nt + 7) >> 3;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int kend = min(2 * (mts[i] + 1), kmax);
            for (int ks = 0; ks < kend; ++ks) {
                const float* ma = sM + (mts[i] * 16 + g) * LDM + ks * 8 + t4;
                const Tf32Val<X3> a[4] = {Tf32Val<X3>(ma[0]), Tf32Val<X3>(ma[8 * LDM]), Tf32Val<X3>(ma[4]),
                                          Tf32Val<X3>(ma[8 * LDM + 4])};
                const float* xb = sX + (ks * 8 + t4) * SSD_LDX + ph * 32 + g;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    mma_x<X3>(acc[i][j], a, Tf32Val<X3>(xb[j * 8]), Tf32Val<X3>(xb[j * 8 + 4 * SSD_LDX]));
            }
        }
    }
    const float dskip = Dv[h];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int t = mts[i] * 16 + g + 8 * r;
            if (t < nt) {
                const float* xr = bc + (ck.row0 + t) * p.conv_dim + h * P + ph * 32 + 2 * t4;
                float* o = y + (ck.row0 + t) * p.d_inner + h * P + ph * 32 + 2 * t4;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 xv = *reinterpret_cast<const float2*>(xr + j * 8);
                    *reinterpret_cast<float2*>(o + j * 8) =
                        make_float2(acc[i][j][2 * r] + dskip * xv.x, acc[i][j][2 * r + 1] + dskip * xv.y);
                }
            }
        }
}

// ===========================================================================
// fp16 forms of the two chunk kernels (fp16 / packed weights only)
// ===========================================================================
// Same algebra with the operands staged as fp16 (11 significant bits like TF32; values
// clamped to the fp16 range, as the activations of the projections around the scan are)
// and read with ldmatrix into mma.sync.m16n8k16 fragments: half the shared memory of the
// TF32 forms (four CTAs per SM instead of two - the kernels are latency-bound, so resident
// warps are what they need) and an eighth of the fragment-load instructions.  Rows are
// padded by 16 bytes so that the eight row addresses of an 8 x 8 ldmatrix tile fall into
// eight different 16-byte bank groups.
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const __half* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const __half* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// four floats -> four clamped halfs, one 8-byte store
__device__ __forceinline__ void store_half4(__half* dst, float4 v) {
    auto cl = [](float x) { return fminf(fmaxf(x, -65504.0f), 65504.0f); };
    const __half2 a = __floats2half2_rn(cl(v.x), cl(v.y)), b = __floats2half2_rn(cl(v.z), cl(v.w));
    *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

constexpr int SSD_LDX16 = SSD_P + 8;       // x tile [Q][P + 8] halfs
constexpr int SSD_LDM16 = SSD_Q + 8;       // M tile [Q][Q + 8] halfs

// As ssd_chunk_state_kernel; d_state a multiple of 32.  S[p][n] = sum_s Xw[s][p] B[s][n]:
// both operands are stored step-major, so both fragments come from transposing loads.
__global__ void __launch_bounds__(SSD_THREADS, 4)
ssd_chunk_state16_kernel(const float* __restrict__ proj, const float* __restrict__ bc, const float* __restrict__ dt_bias,
                         const float* __restrict__ a_log, float* __restrict__ dtcum, float* __restrict__ chunk_state,
                         float* __restrict__ decay, int T, int NC, MambaDims p, const int2* __restrict__ tab, int64_t NT) {
    extern __shared__ __align__(16) uint8_t sm16[];
    constexpr int P = SSD_P;
    const int N = p.d_state, ldb = N + 8;
    __half* sB = reinterpret_cast<__half*>(sm16);      // [Q][N + 8]
    __half* sX = sB + SSD_Q * ldb;                      // [Q][P + 8]   (already multiplied by w_s)
    float* sDt = reinterpret_cast<float*>(sX + SSD_Q * SSD_LDX16);   // [Q]
    float* sCum = sDt + SSD_Q;                          // [Q]
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const SsdChunk ck = ssd_chunk(tab, NT, c, b, h, T, NC, p.n_heads);
    const int nt = ck.nt;
    const float A = -expf(a_log[h]);
    if (threadIdx.x < SSD_Q) {
        float dt = 0.0f;
        if (threadIdx.x < nt) {
            const float u = proj[(ck.row0 + threadIdx.x) * p.proj + p.proj - p.n_heads + h] + dt_bias[h];
            dt = softplus_dt(u);
        }
        sDt[threadIdx.x] = dt;
    }
    __syncthreads();
    if (threadIdx.x < 32) {                 // running sum of A dt over the chunk: 4 steps per lane
        const int l = threadIdx.x;
        float v[4], run = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            run += __fmul_rn(A, sDt[l * 4 + i]);
            v[i] = run;
        }
        float incl = run;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, incl, o);
            if (l >= o) incl += up;
        }
        const float before = incl - run;
#pragma unroll
        for (int i = 0; i < 4; ++i) sCum[l * 4 + i] = before + v[i];
    }
    __syncthreads();
    const float cum_last = sCum[SSD_Q - 1];
    if (threadIdx.x < nt) {
        float* o = dtcum + (ck.dt0 + threadIdx.x) * 2;
        o[0] = sDt[threadIdx.x];
        o[1] = sCum[threadIdx.x];
    }
    if (threadIdx.x == 0) decay[(ck.ci) * p.n_heads + h] = expf(cum_last);
    const int n4 = N >> 2;
    for (int e = threadIdx.x; e < SSD_Q * n4; e += SSD_THREADS) {
        const int t = e / n4, n = (e - t * n4) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < nt) v = *reinterpret_cast<const float4*>(bc + (ck.row0 + t) * p.conv_dim + p.d_inner + n);
        store_half4(sB + t * ldb + n, v);
    }
    for (int e = threadIdx.x; e < SSD_Q * (P / 4); e += SSD_THREADS) {
        const int t = e / (P / 4), i = (e - t * (P / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < nt) {
            const float w = expf(cum_last - sCum[t]) * sDt[t];
            v = *reinterpret_cast<const float4*>(bc + (ck.row0 + t) * p.conv_dim + h * P + i);
            v = make_float4(w * v.x, w * v.y, w * v.z, w * v.w);
        }
        store_half4(sX + t * SSD_LDX16 + i, v);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int mt = warp & 3, nh = warp >> 2;
    const int lj = lane >> 3, lr = lane & 7;            // ldmatrix: which 8 x 8 tile, which of its rows
    const int npairs = N >> 5;                          // pairs of 8-column tiles per half, <= 4
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
    const int ksteps = (nt + 15) >> 4;
    for (int ks = 0; ks < ksteps; ++ks) {
        const int s0 = ks * 16;
        uint32_t a[4];
        ldsm_x4_t(a, sX + (s0 + (lj >> 1) * 8 + lr) * SSD_LDX16 + mt * 16 + (lj & 1) * 8);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
            if (jj < npairs) {
                uint32_t bb[4];
                ldsm_x4_t(bb, sB + (s0 + (lj & 1) * 8 + lr) * ldb + (nh * npairs + jj) * 16 + (lj >> 1) * 8);
                mma_f16(acc[2 * jj], a, bb[0], bb[1]);
                mma_f16(acc[2 * jj + 1], a, bb[2], bb[3]);
            }
    }
    float* out = chunk_state + ((ck.ci) * p.n_heads + h) * P * N;
#pragma unroll
    for (int j = 0; j < 8; ++j)
        if (j < 2 * npairs) {
            const int n = (nh * 2 * npairs + j) * 8 + 2 * t4;
            *reinterpret_cast<float2*>(out + (mt * 16 + g) * N + n) = make_float2(acc[j][0], acc[j][1]);
            *reinterpret_cast<float2*>(out + (mt * 16 + g + 8) * N + n) = make_float2(acc[j][2], acc[j][3]);
        }
}

// As ssd_chunk_out_kernel; d_state a multiple of 16.
__global__ void __launch_bounds__(SSD_THREADS, 4)
ssd_chunk_out16_kernel(const float* __restrict__ bc, const float* __restrict__ G, const float* __restrict__ dtcum,
                       const float* __restrict__ chunk_state, const float* __restrict__ Dv, float* __restrict__ y, int T,
                       int NC, MambaDims p, const int2* __restrict__ tab, int64_t NT) {
    extern __shared__ __align__(16) uint8_t sm16[];
    constexpr int P = SSD_P;
    const int N = p.d_state, ldc = N + 8;
    const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const SsdChunk ck = ssd_chunk(tab, NT, c, b, h, T, NC, p.n_heads);
    const int nt = ck.nt;
    float* sDt = reinterpret_cast<float*>(sm16);        // [Q]
    float* sCum = sDt + SSD_Q;                          // [Q]
    __half* buf = reinterpret_cast<__half*>(sCum + SSD_Q);
    if (threadIdx.x < SSD_Q) {
        float dt = 0.0f, cum = 0.0f;
        if (threadIdx.x < nt) {
            const float2 o = *reinterpret_cast<const float2*>(dtcum + (ck.dt0 + threadIdx.x) * 2);
            dt = o.x;
            cum = o.y;
        }
        sDt[threadIdx.x] = dt;
        sCum[threadIdx.x] = cum;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int lj = lane >> 3, lr = lane & 7;
    const int ph = warp >> 2;
    const int mts[2] = {warp & 3, 7 - (warp & 3)};
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;
    // phase 1: inter-chunk term, A = e^{cum_t} C [t][n] (row-major), B = S_prev [p][n] (row-major)
    {
        __half* sC = buf;                   // [Q][N + 8]
        __half* sS = buf + SSD_Q * ldc;     // [P][N + 8]
        const int n4 = N >> 2;
        for (int e = threadIdx.x; e < SSD_Q * n4; e += SSD_THREADS) {
            const int t = e / n4, n = (e - t * n4) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < nt) {
                const float w = expf(sCum[t]);
                v = *reinterpret_cast<const float4*>(bc + (ck.row0 + t) * p.conv_dim + p.d_inner + N + n);
                v = make_float4(w * v.x, w * v.y, w * v.z, w * v.w);
            }
            store_half4(sC + t * ldc + n, v);
        }
        const float* sp = chunk_state + ((ck.ci) * p.n_heads + h) * P * N;
        for (int e = threadIdx.x; e < P * n4; e += SSD_THREADS) {
            const int i = e / n4, n = (e - i * n4) * 4;
            store_half4(sS + i * ldc + n, __ldcs(reinterpret_cast<const float4*>(sp + i * N + n)));
        }
        __syncthreads();
        for (int ks = 0; ks < (N >> 4); ++ks) {
            const int k0 = ks * 16;
            uint32_t a[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) ldsm_x4(a[i], sC + (mts[i] * 16 + (lj & 1) * 8 + lr) * ldc + k0 + (lj >> 1) * 8);
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                uint32_t bb[4];
                ldsm_x4(bb, sS + (ph * 32 + jj * 16 + (lj >> 1) * 8 + lr) * ldc + k0 + (lj & 1) * 8);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mma_f16(acc[i][2 * jj], a[i], bb[0], bb[1]);
                    mma_f16(acc[i][2 * jj + 1], a[i], bb[2], bb[3]);
                }
            }
        }
    }
    __syncthreads();
    // phase 2: intra-chunk term, A = M [t][s] (row-major), B = x [s][p] (step-major: transposing loads)
    {
        __half* sM = buf;                   // [Q][Q + 8]
        __half* sX = buf + SSD_Q * SSD_LDM16;   // [Q][P + 8]
        const float* gm = G + (ck.ci) * SSD_Q * SSD_Q;
        for (int e = threadIdx.x; e < SSD_Q * (SSD_Q / 4); e += SSD_THREADS) {
            const int t = e / (SSD_Q / 4), s = (e - t * (SSD_Q / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s <= t && t < nt) {
                const float4 gv = *reinterpret_cast<const float4*>(gm + t * SSD_Q + s);
                const float ct = sCum[t];
                v.x = gv.x * expf(ct - sCum[s]) * sDt[s];
                if (s + 1 <= t) v.y = gv.y * expf(ct - sCum[s + 1]) * sDt[s + 1];
                if (s + 2 <= t) v.z = gv.z * expf(ct - sCum[s + 2]) * sDt[s + 2];
                if (s + 3 <= t) v.w = gv.w * expf(ct - sCum[s + 3]) * sDt[s + 3];
            }
            store_half4(sM + t * SSD_LDM16 + s, v);
        }
        for (int e = threadIdx.x; e < SSD_Q * (P / 4); e += SSD_THREADS) {
            const int t = e / (P / 4), i = (e - t * (P / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < nt) v = *reinterpret_cast<const float4*>(bc + (ck.row0 + t) * p.conv_dim + h * P + i);
            store_half4(sX + t * SSD_LDX16 + i, v);
        }
        __syncthreads();
        const int kmax = (nt + 15) >> 4;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int kend = min(mts[i] + 1, kmax);
            for (int ks = 0; ks < kend; ++ks) {
                const int s0 = ks * 16;
                uint32_t a[4];
                ldsm_x4(a, sM + (mts[i] * 16 + (lj & 1) * 8 + lr) * SSD_LDM16 + s0 + (lj >> 1) * 8);
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    uint32_t bb[4];
                    ldsm_x4_t(bb, sX + (s0 + (lj & 1) * 8 + lr) * SSD_LDX16 + ph * 32 + jj * 16 + (lj >> 1) * 8);
                    mma_f16(acc[i][2 * jj], a, bb[0], bb[1]);
                    mma_f16(acc[i][2 * jj + 1], a, bb[2], bb[3]);
                }
            }
        }
    }
    const float dskip = Dv[h];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int t = mts[i] * 16 + g + 8 * r;
            if (t < nt) {
                const float* xr = bc + (ck.row0 + t) * p.conv_dim + h * P + ph * 32 + 2 * t4;
                float* o = y + (ck.row0 + t) * p.d_inner + h * P + ph * 32 + 2 * t4;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 xv = *reinterpret_cast<const float2*>(xr + j * 8);
                    *reinterpret_cast<float2*>(o + j * 8) =
                        make_float2(acc[i][j][2 * r] + dskip * xv.x, acc[i][j][2 * r + 1] + dskip * xv.y);
                }
            }
        }
}

// The chunked scan over proj / bc (as produced by the projection and the convolution):
// y [rows, d_inner], state [B, H, P, N] updated in place.  Rectangular batches: B sequences
// of T steps.  With lay (sequences of different lengths packed back to back, T ignored):
// the chunks of lay's table.  Returns B200_EUNSUPPORTED for shapes outside its tiling (the
// caller then runs the sequential scan).
int mamba_ssd_scan(const float* proj, const float* bc, const float* dt_bias, const float* a_log, const float* D,
                   float* state, float* y, int B, int T, const MambaDims& p, bool precise, const SeqLayout* lay) {
    const int N = p.d_state, P = p.d_head;
    if (P != SSD_P || N % 16 != 0 || N > 128 || (p.d_inner & 3) != 0 || (p.conv_dim & 3) != 0)
        return fail(B200_EUNSUPPORTED, "mamba_ssd_scan: d_head %d / d_state %d outside the chunked kernels' tiling", P, N);
    if (((uintptr_t)bc | (uintptr_t)y) & 15)
        return fail(B200_EUNSUPPORTED, "mamba_ssd_scan: buffers must be 16-byte aligned");
    const int NC = lay ? lay->n_chunks : ceil_div(T, SSD_Q);          // chunks per grid x
    const int64_t chunks = lay ? lay->n_chunks : (int64_t)B * NC;     // entries of the per-chunk arrays
    const int64_t NT = lay ? lay->rows : (int64_t)B * T;
    const int2* tab = lay ? lay->chunks : nullptr;
    const size_t g_f = (size_t)chunks * SSD_Q * SSD_Q, dc_f = (size_t)p.n_heads * NT * 2,
                 cs_f = (size_t)chunks * p.n_heads * P * N, de_f = (size_t)chunks * p.n_heads;
    void* wsp;
    int rc = workspace(WS_ATTN).ensure((g_f + dc_f + cs_f + de_f) * sizeof(float) + 1024, &wsp);
    if (rc) return rc;
    float* G = static_cast<float*>(wsp);
    float* dtcum = G + g_f;
    float* cstate = dtcum + ((dc_f + 3) & ~(size_t)3);
    float* decay = cstate + cs_f;
    const size_t smem_cb = (size_t)SSD_Q * (N + 1) * 4;
    const size_t smem_st = (size_t)(SSD_Q * (N + 8) + SSD_Q * SSD_LDX + 2 * SSD_Q) * 4;
    const size_t smem_out = (size_t)(2 * SSD_Q + std::max(SSD_Q * (N + 4) + P * (N + 4), SSD_Q * (SSD_Q + 4) + SSD_Q * SSD_LDX)) * 4;
    static bool configured = false;
    if (!configured) {
        B200_CUDA(cudaFuncSetAttribute(ssd_cb_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        B200_CUDA(cudaFuncSetAttribute(ssd_chunk_state_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        B200_CUDA(cudaFuncSetAttribute(ssd_chunk_state_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        B200_CUDA(cudaFuncSetAttribute(ssd_chunk_out_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        B200_CUDA(cudaFuncSetAttribute(ssd_chunk_out_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        B200_CUDA(cudaFuncSetAttribute(ssd_chunk_state16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        B200_CUDA(cudaFuncSetAttribute(ssd_chunk_out16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        configured = true;
    }
    B200_REQUIRE(smem_cb <= 160 * 1024 && smem_st <= 160 * 1024 && smem_out <= 160 * 1024, "mamba_ssd_scan: shared memory");
    B200_REQUIRE(NC <= 65535 * 32 && B <= 65535 && p.n_heads <= 65535, "mamba_ssd_scan: grid too large");
    const int gz = lay ? 1 : B;
    // (the upper right quadrant of every G is never written and never read: s <= t only)
    ssd_cb_kernel<<<dim3(3 * NC, gz), SSD_THREADS, smem_cb, stream()>>>(bc, G, T, p, tab);
    B200_LAUNCH_CHECK("ssd_cb_kernel");
    const dim3 grid(NC, p.n_heads, gz);
    const bool half_tiles = !precise && N % 32 == 0;
    const size_t smem_st16 = (size_t)(SSD_Q * (N + 8) + SSD_Q * SSD_LDX16) * 2 + 2 * SSD_Q * 4;
    const size_t smem_out16 = (size_t)std::max(SSD_Q * (N + 8) + P * (N + 8), SSD_Q * SSD_LDM16 + SSD_Q * SSD_LDX16) * 2 + 2 * SSD_Q * 4;
    if (half_tiles)
        ssd_chunk_state16_kernel<<<grid, SSD_THREADS, smem_st16, stream()>>>(proj, bc, dt_bias, a_log, dtcum, cstate, decay, T, NC, p, tab, NT);
    else if (precise)
        ssd_chunk_state_kernel<true><<<grid, SSD_THREADS, smem_st, stream()>>>(proj, bc, dt_bias, a_log, dtcum, cstate, decay, T, NC, p, tab, NT);
    else
        ssd_chunk_state_kernel<false><<<grid, SSD_THREADS, smem_st, stream()>>>(proj, bc, dt_bias, a_log, dtcum, cstate, decay, T, NC, p, tab, NT);
    B200_LAUNCH_CHECK("ssd_chunk_state_kernel");
    ssd_carry_kernel<<<dim3((unsigned)ceil_div(p.d_head * p.d_state, 256), (unsigned)p.n_heads, (unsigned)B), 256, 0, stream()>>>(
        cstate, decay, state, B, NC, p, lay ? lay->seq_chunk0 : nullptr);
    B200_LAUNCH_CHECK("ssd_carry_kernel");
    if (half_tiles)
        ssd_chunk_out16_kernel<<<grid, SSD_THREADS, smem_out16, stream()>>>(bc, G, dtcum, cstate, D, y, T, NC, p, tab, NT);
    else if (precise)
        ssd_chunk_out_kernel<true><<<grid, SSD_THREADS, smem_out, stream()>>>(bc, G, dtcum, cstate, D, y, T, NC, p, tab, NT);
    else
        ssd_chunk_out_kernel<false><<<grid, SSD_THREADS, smem_out, stream()>>>(bc, G, dtcum, cstate, D, y, T, NC, p, tab, NT);
    B200_LAUNCH_CHECK("ssd_chunk_out_kernel");
    return B200_OK;
}

}  // namespace b200
