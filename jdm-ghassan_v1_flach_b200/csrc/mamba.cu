// Mamba-2 layer: single-token state update for decode and the whole-sequence
// forward for prefill.
//
//   projected = in_proj(x)                -> [gate(d_inner) | bc(conv_dim) | dt(n_heads)]
//   bc        = silu(causal depthwise conv_k(bc) + bias)     (window holds RAW inputs)
//   x, B, C   = split(bc)                 (n_groups == 1: B, C are d_state wide)
//   dt        = softplus(dt + dt_bias)    (linear above 20)
//   s         = exp(-exp(A_log) dt) s + (dt B_j) x ;  y = sum_j C_j s_j + D x
//   out       = out_proj(rmsnorm(y * silu(gate)) * norm_w)
//
// Reference arithmetic: core/mamba_cpu.cpp:48-198 (sequence) and the host path of
// Generator::decode_mamba_layer, inference/generator.cpp:510-616 (one token);
// kernels replaced: cuda/mamba.cu:99-345 and :918-1052.
//
// State updates and the convolution use explicit unfused multiply/add in the
// reference's operand order, so given identical inputs the carried state is
// bit-identical to the CPU path; only dot-product summation order differs.
#include "fused.cuh"
#include "gemm.cuh"

namespace b200 {

// ---------------------------------------------------------------------------
// Decode: in_proj GEMV whose epilogue performs the convolution step.
// One warp per projection row, MT sequences per pass.  Rows of the bc section
// read and shift their channel's window [k-1] (oldest first) in place.
// ---------------------------------------------------------------------------
template <int KIND, int MT>
__global__ void __launch_bounds__(GEMV_THREADS)
mamba_inproj_conv_kernel(const float* __restrict__ x, const uint8_t* __restrict__ w_in,
                         const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                         float* __restrict__ conv_state,  // [M, conv_dim, k-1]
                         float* __restrict__ gate,        // [M, d_inner]
                         float* __restrict__ bc,          // [M, conv_dim] (post conv + SiLU)
                         float* __restrict__ dt_raw,      // [M, n_heads]
                         int M, MambaDims p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * GEMV_WARPS + warp;
    if (n >= p.proj) return;
    float acc[MT];
    gemv_row<KIND, MT>(x, w_in, n, M, p.d, lane, acc);
    if (lane >= MT || lane >= M) return;
    // lane m finishes sequence m
    float raw = 0.0f;
#pragma unroll
    for (int m = 0; m < MT; ++m)
        if (m == lane) raw = acc[m];
    const int m = lane;
    if (n < p.d_inner) {
        gate[(int64_t)m * p.d_inner + n] = raw;
    } else if (n < p.d_inner + p.conv_dim) {
        const int c = n - p.d_inner;
        const int win = p.k - 1;
        float* st = conv_state + ((int64_t)m * p.conv_dim + c) * win;
        const float* wc = conv_w + (int64_t)c * p.k;
        float a = conv_b ? conv_b[c] : 0.0f;
        for (int j = 0; j < win; ++j) {
            const float v = st[j];
            a = __fadd_rn(a, __fmul_rn(wc[j], v));
            if (j > 0) st[j - 1] = v;
        }
        a = __fadd_rn(a, __fmul_rn(wc[win], raw));
        if (win > 0) st[win - 1] = raw;
        bc[(int64_t)m * p.conv_dim + c] = silu_acc(a);
    } else {
        dt_raw[(int64_t)m * p.n_heads + (n - p.d_inner - p.conv_dim)] = raw;
    }
}

// ---------------------------------------------------------------------------
// Decode: selective state update.  grid (rows / SCAN_WARPS, M); one warp per state
// row (h, i); lanes stride d_state (coalesced 128-byte accesses).
// ---------------------------------------------------------------------------
constexpr int SCAN_WARPS = 8;
__global__ void __launch_bounds__(SCAN_WARPS * 32)
mamba_step_scan_kernel(const float* __restrict__ bc, const float* __restrict__ dt_raw,
                       const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                       const float* __restrict__ Dv, float* __restrict__ ssm_state,  // [M, rows, d_state]
                       float* __restrict__ y,                                          // [M, d_inner]
                       int dt_stride,                                                  // floats between dt_raw rows
                       MambaDims p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows = p.n_heads * p.d_head;
    const int row = blockIdx.x * SCAN_WARPS + warp;
    const int m = blockIdx.y;
    if (row >= rows) return;
    const int h = row / p.d_head;
    const float u = dt_raw[(int64_t)m * dt_stride + h] + dt_bias[h];
    const float dt = (u > 20.0f) ? u : log1pf(expf(u));
    const float A = -expf(a_log[h]);
    const float dA = expf(__fmul_rn(A, dt));
    const float* bcm = bc + (int64_t)m * p.conv_dim;
    const float xv = bcm[row];
    const float* Bv = bcm + p.d_inner;
    const float* Cv = Bv + p.d_state;
    float* s = ssm_state + ((int64_t)m * rows + row) * p.d_state;
    float acc = 0.0f;
    if (p.d_state == 128) {
        // one 128-bit access per lane covers the row (same products, same order per element)
        float4 sv = *reinterpret_cast<const float4*>(s + lane * 4);
        const float4 b4 = *reinterpret_cast<const float4*>(Bv + lane * 4);
        const float4 c4 = *reinterpret_cast<const float4*>(Cv + lane * 4);
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
    if (lane == 0) y[(int64_t)m * p.d_inner + row] = acc + Dv[h] * xv;
}

// The same update for many sequences (d_state 128, d_head a multiple of SCAN_ROWS): a warp owns
// SCAN_ROWS consecutive rows of one head and issues all their 128-bit state loads before it
// uses any, so that four times the bytes are in flight per warp - with one sequence the
// kernel is a handful of rows per SM, with 64 it is a 200 MB stream that needs them.  Same
// products in the same order per element as the kernel above.
constexpr int SCAN_ROWS = 4;
__global__ void __launch_bounds__(SCAN_WARPS * 32)
mamba_step_scan_stream_kernel(const float* __restrict__ bc, const float* __restrict__ dt_raw,
                              const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                              const float* __restrict__ Dv, float* __restrict__ ssm_state, float* __restrict__ y,
                              int dt_stride, MambaDims p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows = p.n_heads * p.d_head;
    const int row0 = (blockIdx.x * SCAN_WARPS + warp) * SCAN_ROWS;
    const int m = blockIdx.y;
    if (row0 >= rows) return;
    float* s = ssm_state + ((int64_t)m * rows + row0) * 128 + lane * 4;
    float4 sv[SCAN_ROWS];
#pragma unroll
    for (int r = 0; r < SCAN_ROWS; ++r) sv[r] = __ldcs(reinterpret_cast<const float4*>(s + r * 128));
    const int h = row0 / p.d_head;
    const float u = dt_raw[(int64_t)m * dt_stride + h] + dt_bias[h];
    const float dt = (u > 20.0f) ? u : log1pf(expf(u));
    const float A = -expf(a_log[h]);
    const float dA = expf(__fmul_rn(A, dt));
    const float* bcm = bc + (int64_t)m * p.conv_dim;
    const float* Bv = bcm + p.d_inner;
    const float4 b4 = *reinterpret_cast<const float4*>(Bv + lane * 4);
    const float4 c4 = *reinterpret_cast<const float4*>(Bv + 128 + lane * 4);
    const float dskip = Dv[h];
    float acc[SCAN_ROWS], xv[SCAN_ROWS];
#pragma unroll
    for (int r = 0; r < SCAN_ROWS; ++r) {
        xv[r] = bcm[row0 + r];
        float4 v = sv[r];
        v.x = __fadd_rn(__fmul_rn(dA, v.x), __fmul_rn(__fmul_rn(dt, b4.x), xv[r]));
        v.y = __fadd_rn(__fmul_rn(dA, v.y), __fmul_rn(__fmul_rn(dt, b4.y), xv[r]));
        v.z = __fadd_rn(__fmul_rn(dA, v.z), __fmul_rn(__fmul_rn(dt, b4.z), xv[r]));
        v.w = __fadd_rn(__fmul_rn(dA, v.w), __fmul_rn(__fmul_rn(dt, b4.w), xv[r]));
        __stcs(reinterpret_cast<float4*>(s + r * 128), v);
        acc[r] = c4.x * v.x + c4.y * v.y + c4.z * v.z + c4.w * v.w;
    }
#pragma unroll
    for (int r = 0; r < SCAN_ROWS; ++r) acc[r] = warp_sum(acc[r]);
    if (lane < SCAN_ROWS) {
        float a = acc[0], x = xv[0];
#pragma unroll
        for (int r = 1; r < SCAN_ROWS; ++r)
            if (lane == r) { a = acc[r]; x = xv[r]; }
        y[(int64_t)m * p.d_inner + row0 + lane] = a + dskip * x;
    }
}

// ---------------------------------------------------------------------------
// Decode, many sequences: the convolution step on rows of an already computed
// projection [M, proj] (gate | bc | dt).  One thread per (sequence, channel); same
// arithmetic as the epilogue of mamba_inproj_conv_kernel.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
mamba_conv_step_kernel(const float* __restrict__ proj, const float* __restrict__ conv_w,
                       const float* __restrict__ conv_b, float* __restrict__ conv_state, float* __restrict__ bc,
                       int M, MambaDims p) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)M * p.conv_dim) return;
    const int m = (int)(i / p.conv_dim), c = (int)(i - (int64_t)m * p.conv_dim);
    const float raw = proj[(int64_t)m * p.proj + p.d_inner + c];
    const int win = p.k - 1;
    float* st = conv_state + ((int64_t)m * p.conv_dim + c) * win;
    const float* wc = conv_w + (int64_t)c * p.k;
    float a = conv_b ? conv_b[c] : 0.0f;
    for (int j = 0; j < win; ++j) {
        const float v = st[j];
        a = __fadd_rn(a, __fmul_rn(wc[j], v));
        if (j > 0) st[j - 1] = v;
    }
    a = __fadd_rn(a, __fmul_rn(wc[win], raw));
    if (win > 0) st[win - 1] = raw;
    bc[i] = silu_acc(a);
}

// ---------------------------------------------------------------------------
// Gated RMSNorm, one block per row: v = y * silu(gate); out = v / sqrt(mean(v^2)
// + eps) * w with the mean accumulated in double and narrowed to float before
// eps is added (core/mamba_cpu.cpp:176-193).  gate rows are gate_stride apart.
// y may alias out.
// ---------------------------------------------------------------------------
// out16 (optional, with d_inner <= 4096): the result as fp16 rows instead of fp32 (values
// clamped to the fp16 range, as pack_rows_f16 does), for a tensor-core GEMM that follows.
// PER: values of the row a thread keeps in registers (d_inner <= PER * 256), 0 = two passes
// through `out`.  Six CTAs per SM: the kernel is a chain of load -> block reduction -> store
// per row, so resident rows are what hides its latencies.
template <int PER>
__global__ void __launch_bounds__(256, 6)
mamba_gated_norm_kernel(const float* y, const float* __restrict__ gate, int64_t gate_stride,
                        const float* __restrict__ norm_w, float* out, int d_inner, float eps,
                        __half* __restrict__ out16 = nullptr) {
    __shared__ double red[32];
    const int64_t r = blockIdx.x;
    const float* yr = y + r * d_inner;
    const float* gr = gate + r * gate_stride;
    float* o = out + r * d_inner;
    double var = 0.0;
    if (PER > 0) {
        float v[PER > 0 ? PER : 1];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int c = j * 256 + threadIdx.x;
            v[j] = c < d_inner ? yr[c] * silu_acc(gr[c]) : 0.0f;
            var += (double)v[j] * v[j];
        }
        var = block_sum_d(var, red) / (double)d_inner;
        const float inv = 1.0f / sqrtf((float)var + eps);
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int c = j * 256 + threadIdx.x;
            if (c < d_inner) {
                const float res = v[j] * inv * norm_w[c];
                if (out16) out16[r * d_inner + c] = __float2half_rn(fminf(fmaxf(res, -65504.0f), 65504.0f));
                else o[c] = res;
            }
        }
    } else {
        for (int c = threadIdx.x; c < d_inner; c += blockDim.x) {
            const float v = yr[c] * silu_acc(gr[c]);
            o[c] = v;
            var += (double)v * v;
        }
        var = block_sum_d(var, red) / (double)d_inner;
        const float inv = 1.0f / sqrtf((float)var + eps);
        for (int c = threadIdx.x; c < d_inner; c += blockDim.x) o[c] = o[c] * inv * norm_w[c];
    }
}

static void launch_gated_norm(const float* y, const float* gate, int64_t gate_stride, const float* norm_w, float* out,
                              int d_inner, float eps, __half* out16, int64_t rows) {
    const unsigned g = (unsigned)rows;
    if (d_inner <= 1024) mamba_gated_norm_kernel<4><<<g, 256, 0, stream()>>>(y, gate, gate_stride, norm_w, out, d_inner, eps, out16);
    else if (d_inner <= 2048) mamba_gated_norm_kernel<8><<<g, 256, 0, stream()>>>(y, gate, gate_stride, norm_w, out, d_inner, eps, out16);
    else if (d_inner <= 3072) mamba_gated_norm_kernel<12><<<g, 256, 0, stream()>>>(y, gate, gate_stride, norm_w, out, d_inner, eps, out16);
    else if (d_inner <= 4096) mamba_gated_norm_kernel<16><<<g, 256, 0, stream()>>>(y, gate, gate_stride, norm_w, out, d_inner, eps, out16);
    else mamba_gated_norm_kernel<0><<<g, 256, 0, stream()>>>(y, gate, gate_stride, norm_w, out, d_inner, eps, nullptr);
}

// ---------------------------------------------------------------------------
// Prefill: causal depthwise conv + SiLU over [B,T]; the window before t = 0 is
// zero on every call (core/mamba_cpu.cpp:90-99).  One thread per (b,t,c).
// ---------------------------------------------------------------------------
// pos (optional, packed sequences: B = 1, T = all rows): a row's position inside its own
// sequence; taps that would reach before the sequence's first row read zero.
__global__ void mamba_conv_seq_kernel(const float* __restrict__ proj, const float* __restrict__ conv_w,
                                      const float* __restrict__ conv_b, float* __restrict__ bc,
                                      int B, int T, MambaDims p, const int32_t* __restrict__ pos) {
    const int64_t total = (int64_t)B * T * p.conv_dim;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(idx % p.conv_dim);
        const int64_t bt = idx / p.conv_dim;
        const int t = (int)(bt % T);
        const int first = pos ? t - pos[bt] : 0;          // first step of the row's sequence
        const float* wc = conv_w + (int64_t)c * p.k;
        float a = conv_b ? conv_b[c] : 0.0f;
        for (int j = 0; j < p.k; ++j) {
            const int tt = t - (p.k - 1) + j;
            const float v = tt >= first ? proj[(bt - (t - tt)) * p.proj + p.d_inner + c] : 0.0f;
            a = __fadd_rn(a, __fmul_rn(wc[j], v));
        }
        bc[idx] = silu_acc(a);
    }
}

// The same for a window of four taps: a thread owns four adjacent channels and walks
// CONV_TT consecutive steps with the window in registers (one 16-byte load and one
// 16-byte store per step instead of four scalar loads per output).  Same products and
// the same order of additions as the kernel above.
constexpr int CONV_TT = 8;
__global__ void __launch_bounds__(256)
mamba_conv_seq4_kernel(const float* __restrict__ proj, const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                       float* __restrict__ bc, int T, MambaDims p, const int32_t* __restrict__ pos) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= p.conv_dim) return;
    const int t0 = blockIdx.y * CONV_TT, b = blockIdx.z;
    float w[4][4];
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
        const float4 v = *reinterpret_cast<const float4*>(conv_w + (int64_t)(c + ch) * 4);
        w[ch][0] = v.x; w[ch][1] = v.y; w[ch][2] = v.z; w[ch][3] = v.w;
    }
    float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
    if (conv_b) bias = *reinterpret_cast<const float4*>(conv_b + c);
    const float* src = proj + (int64_t)b * T * p.proj + p.d_inner + c;
    auto at = [&](int t) {
        return t >= 0 ? *reinterpret_cast<const float4*>(src + (int64_t)t * p.proj) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    float4 x0 = at(t0 - 3), x1 = at(t0 - 2), x2 = at(t0 - 1);
    float* dst = bc + ((int64_t)b * T + t0) * p.conv_dim + c;
    const int nt = min(CONV_TT, T - t0);
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = 0; i < nt; ++i) {
        const float4 x3 = at(t0 + i);
        if (pos) {
            // packed sequences: the window does not reach into the previous sequence
            const int m = pos[(int64_t)b * T + t0 + i];
            if (m < 3) x0 = zero4;
            if (m < 2) x1 = zero4;
            if (m < 1) x2 = zero4;
        }
        auto tap = [&](float bi, const float (&wc)[4], float a0, float a1, float a2, float a3) {
            float a = __fadd_rn(bi, __fmul_rn(wc[0], a0));
            a = __fadd_rn(a, __fmul_rn(wc[1], a1));
            a = __fadd_rn(a, __fmul_rn(wc[2], a2));
            a = __fadd_rn(a, __fmul_rn(wc[3], a3));
            return silu_acc(a);
        };
        *reinterpret_cast<float4*>(dst + (int64_t)i * p.conv_dim) =
            make_float4(tap(bias.x, w[0], x0.x, x1.x, x2.x, x3.x), tap(bias.y, w[1], x0.y, x1.y, x2.y, x3.y),
                        tap(bias.z, w[2], x0.z, x1.z, x2.z, x3.z), tap(bias.w, w[3], x0.w, x1.w, x2.w, x3.w));
        x0 = x1; x1 = x2; x2 = x3;
    }
}

// ---------------------------------------------------------------------------
// Prefill: sequential selective scan.  One block per (b, h); thread (i, part)
// keeps d_state/PARTS state elements of row i in registers for the whole
// sequence; B_t, C_t are staged through shared memory a tile of timesteps at a
// time.  State is read once and written once.
// ---------------------------------------------------------------------------
constexpr int SEQ_TT = 16;   // timesteps staged per tile
template <int NPT>           // state elements per thread
__global__ void __launch_bounds__(256)
mamba_scan_seq_kernel(const float* __restrict__ proj, const float* __restrict__ bc,
                      const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                      const float* __restrict__ Dv, float* __restrict__ state, float* __restrict__ y,
                      int B, int T, MambaDims p) {
    extern __shared__ float sm[];
    const int parts = p.d_state / NPT;               // threads per row
    const int rows_per_pass = blockDim.x / parts;
    float* sB = sm;                                   // [SEQ_TT][d_state]
    float* sC = sB + SEQ_TT * p.d_state;              // [SEQ_TT][d_state]
    float* sX = sC + SEQ_TT * p.d_state;              // [SEQ_TT][d_head]
    float* sDt = sX + SEQ_TT * p.d_head;              // [SEQ_TT] dt, then [SEQ_TT] dA
    const int b = blockIdx.x / p.n_heads, h = blockIdx.x % p.n_heads;
    const float A = -expf(a_log[h]);
    const float dtb = dt_bias[h];
    const float dskip = Dv[h];
    const int part = threadIdx.x % parts;
    for (int i0 = 0; i0 < p.d_head; i0 += rows_per_pass) {
        const int i = i0 + threadIdx.x / parts;
        const bool active = i < p.d_head;
        float s[NPT];
        float* srow = state + (((int64_t)b * p.n_heads + h) * p.d_head + (active ? i : 0)) * p.d_state + part * NPT;
#pragma unroll
        for (int j = 0; j < NPT; ++j) s[j] = active ? srow[j] : 0.0f;
        for (int t0 = 0; t0 < T; t0 += SEQ_TT) {
            const int nt = min(SEQ_TT, T - t0);
            __syncthreads();
            for (int e = threadIdx.x; e < nt * p.d_state; e += blockDim.x) {
                const int tt = e / p.d_state, j = e % p.d_state;
                const float* brow = bc + ((int64_t)b * T + t0 + tt) * p.conv_dim;
                sB[e] = brow[p.d_inner + j];
                sC[e] = brow[p.d_inner + p.d_state + j];
            }
            for (int e = threadIdx.x; e < nt * p.d_head; e += blockDim.x) {
                const int tt = e / p.d_head, ii = e % p.d_head;
                sX[e] = bc[((int64_t)b * T + t0 + tt) * p.conv_dim + h * p.d_head + ii];
            }
            if (threadIdx.x < nt) {
                const float u = proj[((int64_t)b * T + t0 + threadIdx.x) * p.proj + p.proj - p.n_heads + h] + dtb;
                const float dt = (u > 20.0f) ? u : log1pf(expf(u));
                sDt[threadIdx.x] = dt;
                sDt[SEQ_TT + threadIdx.x] = expf(__fmul_rn(A, dt));
            }
            __syncthreads();
            for (int tt = 0; tt < nt; ++tt) {
                float acc = 0.0f, xv = 0.0f;
                if (active) {
                    const float dt = sDt[tt], dA = sDt[SEQ_TT + tt];
                    xv = sX[tt * p.d_head + i];
                    const float* Bt = sB + tt * p.d_state + part * NPT;
                    const float* Ct = sC + tt * p.d_state + part * NPT;
#pragma unroll
                    for (int j = 0; j < NPT; ++j) {
                        s[j] = __fadd_rn(__fmul_rn(dA, s[j]), __fmul_rn(__fmul_rn(dt, Bt[j]), xv));
                        acc += Ct[j] * s[j];
                    }
                }
                for (int o = parts >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (active && part == 0)
                    y[((int64_t)b * T + t0 + tt) * p.d_inner + h * p.d_head + i] = acc + dskip * xv;
            }
        }
        if (active) {
#pragma unroll
            for (int j = 0; j < NPT; ++j) srow[j] = s[j];
        }
    }
}

// General (slow) scan for shapes the register-resident kernel does not cover:
// one warp per state row, serial over T.
__global__ void mamba_scan_seq_general_kernel(const float* __restrict__ proj, const float* __restrict__ bc,
                                              const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                              const float* __restrict__ Dv, float* __restrict__ state,
                                              float* __restrict__ y, int B, int T, MambaDims p) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int inner = p.n_heads * p.d_head;
    if (warp >= B * inner) return;
    const int b = warp / inner, rem = warp % inner, h = rem / p.d_head;
    const float A = -expf(a_log[h]);
    float* s = state + (int64_t)warp * p.d_state;
    for (int t = 0; t < T; ++t) {
        const float* prow = proj + ((int64_t)b * T + t) * p.proj;
        const float* brow = bc + ((int64_t)b * T + t) * p.conv_dim;
        const float u = prow[p.proj - p.n_heads + h] + dt_bias[h];
        const float dt = (u > 20.0f) ? u : log1pf(expf(u));
        const float dA = expf(__fmul_rn(A, dt));
        const float xv = brow[rem];
        float acc = 0.0f;
        for (int j = lane; j < p.d_state; j += 32) {
            const float sn = __fadd_rn(__fmul_rn(dA, s[j]), __fmul_rn(__fmul_rn(dt, brow[p.d_inner + j]), xv));
            s[j] = sn;
            acc += brow[p.d_inner + p.d_state + j] * sn;
        }
        acc = warp_sum(acc);
        if (lane == 0) y[((int64_t)b * T + t) * p.d_inner + rem] = acc + Dv[h] * xv;
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
static int check_dims(const char* who, const MambaDims& p) {
    B200_REQUIRE(p.d > 0 && p.d_inner > 0 && p.n_heads > 0 && p.d_head > 0 && p.d_state > 0 && p.k >= 1,
                 "%s: bad dims", who);
    B200_REQUIRE(p.d_inner == p.n_heads * p.d_head, "%s: d_inner must equal n_heads*d_head", who);
    // n_groups == 1 only, like the reference's device kernels (cuda/mamba.cu:189-190)
    B200_REQUIRE(p.conv_dim == p.d_inner + 2 * p.d_state, "%s: conv_dim must be d_inner + 2*d_state (n_groups == 1)", who);
    B200_REQUIRE(p.d % 32 == 0 && p.d_inner % 32 == 0, "%s: d and d_inner must be multiples of 32", who);
    return B200_OK;
}

template <int KIND>
static int launch_inproj_conv(const float* x, const uint8_t* w_in, const float* conv_w, const float* conv_b,
                              float* conv_state, float* gate, float* bc, float* dt_raw, int M, const MambaDims& p) {
    const int grid = ceil_div(p.proj, GEMV_WARPS);
    if (M == 1) mamba_inproj_conv_kernel<KIND, 1><<<grid, GEMV_THREADS, 0, stream()>>>(x, w_in, conv_w, conv_b, conv_state, gate, bc, dt_raw, M, p);
    else if (M == 2) mamba_inproj_conv_kernel<KIND, 2><<<grid, GEMV_THREADS, 0, stream()>>>(x, w_in, conv_w, conv_b, conv_state, gate, bc, dt_raw, M, p);
    else if (M <= 4) mamba_inproj_conv_kernel<KIND, 4><<<grid, GEMV_THREADS, 0, stream()>>>(x, w_in, conv_w, conv_b, conv_state, gate, bc, dt_raw, M, p);
    else mamba_inproj_conv_kernel<KIND, 8><<<grid, GEMV_THREADS, 0, stream()>>>(x, w_in, conv_w, conv_b, conv_state, gate, bc, dt_raw, M, p);
    B200_LAUNCH_CHECK("mamba_inproj_conv_kernel");
    return B200_OK;
}

// kind: template tag (KIND_F32, KIND_F16, 0..3)
int mamba2_step(const float* x, const void* w_in, const float* conv_w, const float* conv_b,
                const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                const void* w_out, float* conv_state, float* ssm_state, float* out, int batch,
                MambaDims p, int kind) {
    if (batch <= 0) return B200_OK;
    int rc = check_dims("mamba2_step", p);
    if (rc) return rc;
    B200_REQUIRE(x && w_in && conv_w && dt_bias && a_log && D && norm_w && w_out && conv_state && ssm_state && out,
                 "mamba2_step: null pointer");
    if (kind >= 0 && kind <= 3)
        B200_REQUIRE(p.d % q_block_elems(kind) == 0 && p.d_inner % q_block_elems(kind) == 0,
                     "mamba2_step: d and d_inner must be multiples of the quantisation block");
    p.proj = p.d_inner + p.conv_dim + p.n_heads;
    // workspace: gate | bc | dt_raw | y   per sequence
    const size_t per = (size_t)p.d_inner * 2 + p.conv_dim + p.n_heads;
    void* wsp;
    rc = workspace(WS_MAMBA).ensure(per * batch * sizeof(float) + 256, &wsp);
    if (rc) return rc;
    float* gate = static_cast<float*>(wsp);
    float* bc = gate + (size_t)batch * p.d_inner;
    float* dt_raw = bc + (size_t)batch * p.conv_dim;
    float* y = dt_raw + (((size_t)batch * p.n_heads + 3) & ~(size_t)3);
    const int win = p.k - 1;
    const int rows = p.n_heads * p.d_head;
    if (batch >= GEMM_MIN_ROWS && kind != KIND_F32) {
        // many sequences: both projections as tensor-core GEMMs, the conv step on its own
        void* wsp2;
        const bool out_gemm = p.d_inner % 8 == 0 && p.d_inner <= 4096 && linear_uses_gemm(w_out, kind, out, batch, p.d_inner, p.d);
        const size_t f32_bytes = ((per + p.proj) * batch * sizeof(float) + 255) & ~(size_t)255;
        rc = workspace(WS_MAMBA).ensure(f32_bytes + (out_gemm ? (size_t)batch * p.d_inner * 2 : 0) + 512, &wsp2);
        if (rc) return rc;
        gate = static_cast<float*>(wsp2);
        bc = gate + (size_t)batch * p.d_inner;
        dt_raw = bc + (size_t)batch * p.conv_dim;
        y = dt_raw + (((size_t)batch * p.n_heads + 3) & ~(size_t)3);
        float* proj = y + (size_t)batch * p.d_inner;
        __half* y16 = reinterpret_cast<__half*>(static_cast<char*>(wsp2) + f32_bytes);   // the normed rows for out_proj
        rc = linear(x, w_in, kind, proj, batch, p.d, p.proj);
        if (rc) return rc;
        const int64_t items = (int64_t)batch * p.conv_dim;
        mamba_conv_step_kernel<<<(unsigned)ceil_div64(items, 256), 256, 0, stream()>>>(proj, conv_w, conv_b, conv_state,
                                                                                       bc, batch, p);
        B200_LAUNCH_CHECK("mamba_conv_step_kernel");
        if (p.d_state == 128 && p.d_head % SCAN_ROWS == 0 && (reinterpret_cast<uintptr_t>(ssm_state) & 15) == 0 &&
            (reinterpret_cast<uintptr_t>(bc) & 15) == 0 && p.conv_dim % 4 == 0 && p.d_inner % 4 == 0)
            mamba_step_scan_stream_kernel<<<dim3(ceil_div(rows, SCAN_WARPS * SCAN_ROWS), batch), SCAN_WARPS * 32, 0, stream()>>>(
                bc, proj + p.d_inner + p.conv_dim, dt_bias, a_log, D, ssm_state, y, p.proj, p);
        else
            mamba_step_scan_kernel<<<dim3(ceil_div(rows, SCAN_WARPS), batch), SCAN_WARPS * 32, 0, stream()>>>(
                bc, proj + p.d_inner + p.conv_dim, dt_bias, a_log, D, ssm_state, y, p.proj, p);
        B200_LAUNCH_CHECK("mamba_step_scan_kernel");
        launch_gated_norm(y, proj, p.proj, norm_w, y, p.d_inner, p.eps, out_gemm ? y16 : nullptr, batch);
        B200_LAUNCH_CHECK("mamba_gated_norm_kernel");
        if (out_gemm) return linear_a16(y16, w_out, kind, out, batch, p.d_inner, p.d);
        return linear(y, w_out, kind, out, batch, p.d_inner, p.d);
    }
    for (int m0 = 0; m0 < batch; m0 += 8) {
        const int M = std::min(8, batch - m0);
        const float* xm = x + (int64_t)m0 * p.d;
        float* cs = conv_state + (int64_t)m0 * p.conv_dim * win;
        float* g = gate + (int64_t)m0 * p.d_inner;
        float* b = bc + (int64_t)m0 * p.conv_dim;
        float* dtr = dt_raw + (int64_t)m0 * p.n_heads;
        const uint8_t* wi = static_cast<const uint8_t*>(w_in);
        switch (kind) {
            case 0: rc = launch_inproj_conv<0>(xm, wi, conv_w, conv_b, cs, g, b, dtr, M, p); break;
            case 1: rc = launch_inproj_conv<1>(xm, wi, conv_w, conv_b, cs, g, b, dtr, M, p); break;
            case 2: rc = launch_inproj_conv<2>(xm, wi, conv_w, conv_b, cs, g, b, dtr, M, p); break;
            case 3: rc = launch_inproj_conv<3>(xm, wi, conv_w, conv_b, cs, g, b, dtr, M, p); break;
            case KIND_F16: rc = launch_inproj_conv<KIND_F16>(xm, wi, conv_w, conv_b, cs, g, b, dtr, M, p); break;
            default: rc = launch_inproj_conv<KIND_F32>(xm, wi, conv_w, conv_b, cs, g, b, dtr, M, p); break;
        }
        if (rc) return rc;
    }
    mamba_step_scan_kernel<<<dim3(ceil_div(rows, SCAN_WARPS), batch), SCAN_WARPS * 32, 0, stream()>>>(
        bc, dt_raw, dt_bias, a_log, D, ssm_state, y, p.n_heads, p);
    B200_LAUNCH_CHECK("mamba_step_scan_kernel");
    launch_gated_norm(y, gate, p.d_inner, norm_w, y, p.d_inner, p.eps, nullptr, batch);
    B200_LAUNCH_CHECK("mamba_gated_norm_kernel");
    return linear(y, w_out, kind, out, batch, p.d_inner, p.d);
}

// mamba_ssd.cu
int mamba_ssd_scan(const float* proj, const float* bc, const float* dt_bias, const float* a_log, const float* D,
                   float* state, float* y, int B, int T, const MambaDims& p, bool precise, const SeqLayout* lay);
constexpr int SSD_MIN_STEPS = 64;

// The last k-1 raw (pre-convolution) inputs of every channel, oldest first: the window a
// decode step expects after this sequence (zeros where the sequence is shorter).
__global__ void mamba_conv_window_kernel(const float* __restrict__ proj, float* __restrict__ conv_state, int B, int T,
                                         MambaDims p, const int32_t* __restrict__ seq_off) {
    const int win = p.k - 1;
    const int64_t total = (int64_t)B * p.conv_dim * win;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int j = (int)(i % win);
        const int64_t bc_i = i / win;
        const int c = (int)(bc_i % p.conv_dim), b = (int)(bc_i / p.conv_dim);
        const int64_t first = seq_off ? seq_off[b] : (int64_t)b * T;
        const int len = seq_off ? seq_off[b + 1] - seq_off[b] : T;
        const int t = len - win + j;
        conv_state[i] = t >= 0 ? proj[(first + t) * p.proj + p.d_inner + c] : 0.0f;
    }
}

int mamba2_forward(const float* x, const void* w_in, const float* conv_w, const float* conv_b,
                   const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                   const void* w_out, float* state, float* out, int B, int T, MambaDims p, int kind,
                   float* conv_state_out, const void* x16, const SeqLayout* lay) {
    if (lay) {
        B200_REQUIRE(lay->n_seq == B && lay->rows > 0 && lay->seq_off && lay->pos && lay->host_off,
                     "mamba2_forward: incomplete sequence layout");
        T = 1;
    }
    if (B <= 0 || T <= 0) return B200_OK;
    int rc = check_dims("mamba2_forward", p);
    if (rc) return rc;
    B200_REQUIRE(x && w_in && conv_w && dt_bias && a_log && D && norm_w && w_out && state && out,
                 "mamba2_forward: null pointer");
    p.proj = p.d_inner + p.conv_dim + p.n_heads;
    const int64_t NT = lay ? lay->rows : (int64_t)B * T;
    B200_REQUIRE(NT <= 0x7fffffff, "mamba2_forward: B*T too large");
    // the convolution sees packed sequences as one long one whose rows know their position
    const int cB = lay ? 1 : B, cT = lay ? (int)NT : T;
    const int32_t* pos = lay ? lay->pos : nullptr;
    const size_t proj_f = (size_t)NT * p.proj, bc_f = (size_t)NT * p.conv_dim, y_f = (size_t)NT * p.d_inner;
    void* wsp;
    // when the out-projection runs as a GEMM the gated norm hands it fp16 rows directly
    const bool out_gemm = p.d_inner <= 4096 && linear_uses_gemm(w_out, kind, out, (int)NT, p.d_inner, p.d);
    const size_t y16_f = out_gemm ? (y_f + 1) / 2 : 0;                      // fp16 rows, counted in floats
    rc = workspace(WS_MAMBA).ensure((proj_f + bc_f + y_f + y16_f) * sizeof(float) + 1024, &wsp);
    if (rc) return rc;
    float* proj = static_cast<float*>(wsp);
    float* bc = proj + ((proj_f + 3) & ~(size_t)3);
    float* y = bc + ((bc_f + 3) & ~(size_t)3);
    __half* y16 = reinterpret_cast<__half*>(y + ((y_f + 3) & ~(size_t)3));
    if (x16 && linear_uses_gemm(w_in, kind, proj, (int)NT, p.d, p.proj) && (reinterpret_cast<uintptr_t>(x16) & 15) == 0)
        rc = linear_a16(x16, w_in, kind, proj, (int)NT, p.d, p.proj);
    else
        rc = linear(x, w_in, kind, proj, (int)NT, p.d, p.proj);
    if (rc) return rc;
    {
        const int64_t total = NT * p.conv_dim;
        const int grid = (int)std::min<int64_t>(ceil_div64(total, 256), (int64_t)num_sms() * 32);
        auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
        if (p.k == 4 && p.conv_dim % 4 == 0 && p.d_inner % 4 == 0 && p.proj % 4 == 0 && al16(proj) && al16(bc) &&
            al16(conv_w) && (!conv_b || al16(conv_b)) && cB <= 65535 && ceil_div(cT, CONV_TT) <= 65535) {
            mamba_conv_seq4_kernel<<<dim3(ceil_div(p.conv_dim / 4, 256), ceil_div(cT, CONV_TT), cB), 256, 0, stream()>>>(
                proj, conv_w, conv_b, bc, cT, p, pos);
            B200_LAUNCH_CHECK("mamba_conv_seq4_kernel");
        } else {
            mamba_conv_seq_kernel<<<grid, 256, 0, stream()>>>(proj, conv_w, conv_b, bc, cB, cT, p, pos);
            B200_LAUNCH_CHECK("mamba_conv_seq_kernel");
        }
        if (conv_state_out && p.k > 1) {
            const int64_t n = (int64_t)B * p.conv_dim * (p.k - 1);
            mamba_conv_window_kernel<<<(unsigned)std::min<int64_t>(ceil_div64(n, 256), 4096), 256, 0, stream()>>>(
                proj, conv_state_out, B, T, p, lay ? lay->seq_off : nullptr);
            B200_LAUNCH_CHECK("mamba_conv_window_kernel");
        }
    }
    // Long sequences: the chunked form (all steps in parallel, a short carry over chunks);
    // short ones and shapes outside its tiling: the sequential register-resident scan.
    bool scanned = false;
    if (lay ? lay->chunks != nullptr : T >= SSD_MIN_STEPS) {
        rc = mamba_ssd_scan(proj, bc, dt_bias, a_log, D, state, y, B, T, p, kind == KIND_F32, lay);
        if (rc == B200_OK) scanned = true;
        else if (rc != B200_EUNSUPPORTED) return rc;
    }
    // the sequential scan of `nb` equally long sequences starting at row `row0`
    auto sequential = [&](int64_t row0, int nb, int steps, float* st) -> int {
        const float* pj = proj + row0 * p.proj;
        const float* bcs = bc + row0 * p.conv_dim;
        float* ys = y + row0 * p.d_inner;
        // register-resident scan: 256 threads = rows_per_pass * parts, parts a power of two <= 32
        int npt = 0;
        for (int cand : {32, 16, 8, 4}) {
            const int parts = p.d_state / cand;
            if (p.d_state % cand == 0 && parts >= 1 && parts <= 32 && (parts & (parts - 1)) == 0 && 256 % parts == 0) {
                npt = cand;
                break;
            }
        }
        const size_t smem = (size_t)SEQ_TT * (2 * p.d_state + p.d_head + 2) * sizeof(float);
        if (npt && smem <= 48 * 1024) {
            const int grid = nb * p.n_heads;
            if (npt == 32) mamba_scan_seq_kernel<32><<<grid, 256, smem, stream()>>>(pj, bcs, dt_bias, a_log, D, st, ys, nb, steps, p);
            else if (npt == 16) mamba_scan_seq_kernel<16><<<grid, 256, smem, stream()>>>(pj, bcs, dt_bias, a_log, D, st, ys, nb, steps, p);
            else if (npt == 8) mamba_scan_seq_kernel<8><<<grid, 256, smem, stream()>>>(pj, bcs, dt_bias, a_log, D, st, ys, nb, steps, p);
            else mamba_scan_seq_kernel<4><<<grid, 256, smem, stream()>>>(pj, bcs, dt_bias, a_log, D, st, ys, nb, steps, p);
            B200_LAUNCH_CHECK("mamba_scan_seq_kernel");
        } else {
            const int64_t warps = (int64_t)nb * p.n_heads * p.d_head;
            mamba_scan_seq_general_kernel<<<(unsigned)ceil_div64(warps * 32, 256), 256, 0, stream()>>>(
                pj, bcs, dt_bias, a_log, D, st, ys, nb, steps, p);
            B200_LAUNCH_CHECK("mamba_scan_seq_general_kernel");
        }
        return B200_OK;
    };
    if (!scanned && !lay) {
        rc = sequential(0, B, T, state);
        if (rc) return rc;
    } else if (!scanned) {
        // packed sequences on a shape outside the chunked kernels: one scan per sequence
        for (int b = 0; b < B; ++b) {
            rc = sequential(lay->host_off[b], 1, lay->host_off[b + 1] - lay->host_off[b],
                            state + (int64_t)b * p.d_inner * p.d_state);
            if (rc) return rc;
        }
    }
    launch_gated_norm(y, proj, p.proj, norm_w, y, p.d_inner, p.eps, out_gemm ? y16 : nullptr, NT);
    B200_LAUNCH_CHECK("mamba_gated_norm_kernel");
    if (out_gemm) return linear_a16(y16, w_out, kind, out, (int)NT, p.d_inner, p.d);
    return linear(y, w_out, kind, out, (int)NT, p.d_inner, p.d);
}

}  // namespace b200

using namespace b200;

static MambaDims dims_of(int d, int d_inner, int conv_dim, int n_heads, int d_head, int d_state, int k, float eps) {
    MambaDims p;
    p.d = d; p.d_inner = d_inner; p.conv_dim = conv_dim; p.n_heads = n_heads; p.d_head = d_head;
    p.d_state = d_state; p.k = k; p.eps = eps; p.proj = d_inner + conv_dim + n_heads;
    return p;
}

extern "C" {

int b200_mamba2_forward(const float* x, const float* w_in, const float* conv_w, const float* conv_b,
                        const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                        const float* w_out, float* state, float* out, int B, int T, int d, int d_inner,
                        int conv_dim, int n_heads, int d_head, int d_state, int k, float eps) {
    return mamba2_forward(x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, state, out, B, T,
                          dims_of(d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps), KIND_F32);
}
int b200_mamba2_forward_half(const float* x, const uint16_t* w_in, const float* conv_w, const float* conv_b,
                             const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                             const uint16_t* w_out, float* state, float* out, int B, int T, int d, int d_inner,
                             int conv_dim, int n_heads, int d_head, int d_state, int k, float eps, int qkind) {
    B200_REQUIRE(qkind >= -1 && qkind <= 3, "mamba2_forward_half: unknown qkind %d", qkind);
    return mamba2_forward(x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, state, out, B, T,
                          dims_of(d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps), tag_of_qkind(qkind));
}
int b200_mamba2_step(const float* x, const float* w_in, const float* conv_w, const float* conv_b,
                     const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                     const float* w_out, float* conv_state, float* ssm_state, float* out,
                     int d, int d_inner, int conv_dim, int n_heads, int d_head, int d_state, int k, float eps) {
    return mamba2_step(x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, conv_state, ssm_state, out, 1,
                       dims_of(d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps), KIND_F32);
}
int b200_mamba2_step_half(const float* x, const uint16_t* w_in, const float* conv_w, const float* conv_b,
                          const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                          const uint16_t* w_out, float* conv_state, float* ssm_state, float* out,
                          int d, int d_inner, int conv_dim, int n_heads, int d_head, int d_state, int k,
                          float eps, int qkind) {
    B200_REQUIRE(qkind >= -1 && qkind <= 3, "mamba2_step_half: unknown qkind %d", qkind);
    return mamba2_step(x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, conv_state, ssm_state, out, 1,
                       dims_of(d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps), tag_of_qkind(qkind));
}
int b200_mamba2_step_batched(const float* x, const uint16_t* w_in, const float* conv_w, const float* conv_b,
                             const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                             const uint16_t* w_out, float* conv_state, float* ssm_state, float* out,
                             int batch, int d, int d_inner, int conv_dim, int n_heads, int d_head,
                             int d_state, int k, float eps, int qkind) {
    B200_REQUIRE(qkind >= -1 && qkind <= 3, "mamba2_step_batched: unknown qkind %d", qkind);
    return mamba2_step(x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, conv_state, ssm_state, out, batch,
                       dims_of(d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps), tag_of_qkind(qkind));
}

}  // extern "C"
