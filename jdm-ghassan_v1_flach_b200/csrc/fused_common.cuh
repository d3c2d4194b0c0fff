// Device-side machinery shared by the fused decode-step kernels: the TMA ring, the
// staging of activations in shared memory, the per-tile dot products (tensor-core
// path for Q4_K and fp16 weights, scalar path for the 32-element formats and fp32)
// and the launch helpers.
//
// Kernel shape: SG_CONSUMERS consumer warps + one producer warp.  The producer
// streams weight tiles (<= 16 rows, contiguous bytes) into a ring of stages; the
// consumers compute the tile's dot products into a small shared buffer
// red[buf][part][pass][row][token]; after one consumer barrier the threads
// (row, token) add the parts and run the epilogue.  `pass` lets one tile carry two
// matrices (gate and up rows of the same expert).
#pragma once

#include "fused.cuh"
#include "mma_tile.cuh"

namespace b200 {

constexpr int SG_CONSUMERS = 8;                    // consumer warps
constexpr int SG_CTHREADS = SG_CONSUMERS * 32;
constexpr int SG_THREADS = SG_CTHREADS + 32;       // + one producer warp
constexpr int SG_MAX_STAGES = 4;
constexpr int SMEM_BUDGET = 113 * 1024;            // per CTA: two kernels' CTAs fit one SM, so a
                                                   // dependent kernel can start streaming early
constexpr int SMEM_BUDGET_FULL = 200 * 1024;       // fallback for wide rows: one CTA per SM
constexpr int TILE_ROWS = 16;                      // rows of a tile on the tensor-core path (max elsewhere)
constexpr int RED_TOK = 8;                         // token columns
constexpr int RED_PASS = TILE_ROWS * RED_TOK;      // floats of one (part, pass)
constexpr int RED_PASSES = 2;
constexpr int RED_BUF = SG_CONSUMERS * RED_PASSES * RED_PASS;   // floats of one buffer
constexpr int RED_FLOATS = 2 * RED_BUF;                         // double-buffered by tile parity
constexpr int BAR_BYTES = 2 * SG_MAX_STAGES * 8 + 2 * SG_CONSUMERS * 8;   // mbarriers + reduction scratch

template <int KIND>
struct UsesMma {
    static constexpr bool value = (KIND == 3 || KIND == KIND_F16);
};

#ifdef __CUDACC__
// NC consumer warps (the default is the fused per-phase kernels' count; the persistent
// step kernel runs more).
template <int NC = SG_CONSUMERS>
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NC * 32) : "memory"); }

// Sum over the consumer threads; result in every consumer thread.  red: >= SG_CONSUMERS doubles.
__device__ __forceinline__ double consumer_sum_d(double v, double* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    v = warp_sum_d(v);
    consumer_sync<>();
    if (lane == 0) red[wid] = v;
    consumer_sync<>();
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < SG_CONSUMERS; ++w) t += red[w];
    return t;
}

// ---- the shared-memory ring ---------------------------------------------------
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
    // i / n_stages and i % n_stages without a division (n_stages <= SG_MAX_STAGES = 4: the high
    // word of i * ceil(2^32 / n) is the exact quotient for every i below 2^31)
    __device__ __forceinline__ int lap(int i) const {
        const uint32_t inv = n_stages == 2 ? 0x80000000u : n_stages == 3 ? 0x55555556u : 0x40000000u;
        return n_stages == 1 ? i : (int)__umulhi((uint32_t)i, inv);
    }
    __device__ __forceinline__ int slot(int i) const { return i - lap(i) * n_stages; }
    __device__ __forceinline__ uint8_t* stage(int i) const { return stages + (size_t)slot(i) * stage_bytes; }
    // producer side
    __device__ __forceinline__ bool acquire(int i) {
        return i < n_stages || mbar_wait(&empty[slot(i)], (lap(i) - 1) & 1, status);
    }
    __device__ __forceinline__ void expect(int i, uint32_t bytes) { mbar_expect_tx(&full[slot(i)], bytes); }
    __device__ __forceinline__ void copy(int i, int offset, const void* src, uint32_t bytes) {
        tma_load_1d(stage(i) + offset, src, bytes, &full[slot(i)]);
    }
    // never leave with copies of this CTA still in flight
    __device__ __forceinline__ void drain(int issued) {
        for (int i = max(0, issued - n_stages); i < issued; ++i)
            if (!mbar_wait(&full[slot(i)], lap(i) & 1, status)) break;
    }
    // consumer side
    __device__ __forceinline__ bool wait_full(int i) { return mbar_wait(&full[slot(i)], lap(i) & 1, status); }
    __device__ __forceinline__ void release(int i) {
        __syncwarp();
        if ((threadIdx.x & 31) == 0) mbar_arrive(&empty[slot(i)]);
    }
};
static_assert(SG_MAX_STAGES <= 4, "Ring::lap covers up to four stages");

// ---- activations in shared memory ----------------------------------------------
// Scalar path: fp32, unit-major (stream.cuh).  Tensor-core path: fp16 hi/lo parts
// and sub-block sums (mma_tile.cuh), plus an optional fp32 copy in natural order
// (needed while normalising and by the exact-order router).
struct XAct {
    float* xs = nullptr;       // scalar path: [tokens][xs_tok]
    int xs_tok = 0;
    __half *hi = nullptr, *lo = nullptr;   // tensor-core path
    float* sumx = nullptr;
    float* f32 = nullptr;      // [tokens][K] natural order, may be null
    int K = 0, tokens = 0;
    int zrow = -1;             // row that stands in for absent tokens (-1: the zero row after the last token)
    __device__ __forceinline__ XHalf half() const {
        XHalf h;
        h.hi = hi; h.lo = lo; h.sumx = sumx; h.stride = K + XH_PAD; h.nsub = K >> 5; h.zero_row = zrow >= 0 ? zrow : tokens;
        return h;
    }
};

template <int KIND>
__host__ __device__ inline size_t xact_bytes(int K, int tokens, bool want_f32) {
    if (UsesMma<KIND>::value) return xhalf_bytes(K, tokens) + 16 + (want_f32 ? (size_t)tokens * K * 4 : 0);
    return (size_t)tokens * xs_floats(K) * 4;
}

// Carve an XAct out of shared memory at p (16-byte aligned); returns the end.
template <int KIND>
__device__ __forceinline__ uint8_t* xact_carve(XAct& xa, uint8_t* p, int K, int tokens, bool want_f32) {
    xa.K = K;
    xa.tokens = tokens;
    if (UsesMma<KIND>::value) {
        const size_t row = (size_t)(K + XH_PAD);
        xa.hi = reinterpret_cast<__half*>(p);
        xa.lo = xa.hi + (size_t)(tokens + 1) * row;
        xa.sumx = reinterpret_cast<float*>(xa.lo + (size_t)(tokens + 1) * row);
        p = reinterpret_cast<uint8_t*>(xa.sumx + (size_t)(tokens + 1) * (K >> 5));
        p = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 15) & ~(uintptr_t)15);
        if (want_f32) {
            xa.f32 = reinterpret_cast<float*>(p);
            p += (size_t)tokens * K * 4;
        }
    } else {
        xa.xs = reinterpret_cast<float*>(p);
        xa.xs_tok = xs_floats(K);
        p += (size_t)tokens * xa.xs_tok * 4;
    }
    return p;
}

// Zero row of the tensor-core layout (stands in for tokens beyond M).
template <int KIND, int NC = SG_CONSUMERS>
__device__ __forceinline__ void xact_zero_row(const XAct& xa) {
    constexpr int SG_CTHREADS = NC * 32;
    if (UsesMma<KIND>::value) {
        const size_t row = (size_t)(xa.K + XH_PAD);
        for (int k = threadIdx.x; k < xa.K + XH_PAD; k += SG_CTHREADS) {
            xa.hi[(size_t)xa.tokens * row + k] = __ushort_as_half(0);
            xa.lo[(size_t)xa.tokens * row + k] = __ushort_as_half(0);
        }
        for (int s = threadIdx.x; s < (xa.K >> 5); s += SG_CTHREADS) xa.sumx[(size_t)xa.tokens * (xa.K >> 5) + s] = 0.0f;
    }
}

__device__ __forceinline__ void split_half(float v, __half& h, __half& l) {
    v = fminf(fmaxf(v, -60000.0f), 60000.0f);
    h = __float2half_rn(v);
    l = __float2half_rn(v - __half2float(h));
}

// Two sums over the consumer threads at once; red: >= 2 * NC doubles.
template <int NC = SG_CONSUMERS>
__device__ __forceinline__ void consumer_sum_d2(double& a, double& b, double* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    a = warp_sum_d(a);
    b = warp_sum_d(b);
    consumer_sync<NC>();
    if (lane == 0) { red[wid] = a; red[NC + wid] = b; }
    consumer_sync<NC>();
    a = 0.0;
    b = 0.0;
#pragma unroll
    for (int w = 0; w < NC; ++w) { a += red[w]; b += red[NC + w]; }
}

// Token m's activations from global memory (K floats at x) into shared memory.
// A thread owns runs of four consecutive k (one 128-bit load each) and keeps them in
// registers across the reduction, so global memory is read once, every load is in
// flight before the first is used, and one barrier (three with a reduction)
// separates load from use.  Eight neighbouring lanes hold one 32-wide sub-block, so
// the sub-block sums of the tensor-core path take three shuffles.
// RMS: v = x * inv_rms * norm_w in the reference's operand order
// (core/math_cpu.cpp:299-316; inv from a double sum of squares); nw_s is norm_w
// already in shared memory.  `extra` is summed over the consumer threads in the same
// reduction and returned (used for the gated-norm partial sums).  Consumer threads
// only; ends with a consumer barrier.  K % 32 == 0.
// CG: x was written by other CTAs of the running kernel (persistent step kernel): every
// load goes to L2 (ld.global.cg) so that no stale L1 line is read.
constexpr int XQ_REG = 4;                          // runs per thread held in registers: K <= 4096
template <bool CG>
__device__ __forceinline__ float4 ld_f4(const float* p) {
    return CG ? __ldcg(reinterpret_cast<const float4*>(p)) : *reinterpret_cast<const float4*>(p);
}
template <bool CG>
__device__ __forceinline__ float ld_f1(const float* p) { return CG ? __ldcg(p) : *p; }
template <int KIND, bool RMS, bool EXTRA, bool CG = false, int NC = SG_CONSUMERS>
__device__ __forceinline__ double stage_x(const float* x, const float* nw_s, const XAct& xa, int m,
                                          float eps, double* red, double extra) {
    constexpr int SG_CTHREADS = NC * 32;
    const int K = xa.K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* xs = UsesMma<KIND>::value ? nullptr : xa.xs + (size_t)m * xa.xs_tok;
    const size_t row = (size_t)(K + XH_PAD);
    __half* hi = UsesMma<KIND>::value ? xa.hi + (size_t)m * row : nullptr;
    __half* lo = UsesMma<KIND>::value ? xa.lo + (size_t)m * row : nullptr;
    float* f32 = (UsesMma<KIND>::value && xa.f32) ? xa.f32 + (size_t)m * K : nullptr;
    float* sx = UsesMma<KIND>::value ? xa.sumx + (size_t)m * (K >> 5) : nullptr;
    const int nq = K >> 2;                                          // runs of four
    const int nrun = (nq + SG_CTHREADS - 1) / SG_CTHREADS;
    if (nrun <= XQ_REG && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        // final values of run q (k = 4q .. 4q+3); every lane of the warp calls this
        auto emit4 = [&](int q, bool ok, float4 v) {
            const int k = q << 2;
            if (UsesMma<KIND>::value) {
                __half h[4], l[4];
                split_half(v.x, h[0], l[0]);
                split_half(v.y, h[1], l[1]);
                split_half(v.z, h[2], l[2]);
                split_half(v.w, h[3], l[3]);
                float t = 0.0f;
#pragma unroll
                for (int e = 0; e < 4; ++e) t += __half2float(h[e]) + __half2float(l[e]);
                if (!ok) t = 0.0f;
                t += __shfl_xor_sync(0xffffffffu, t, 1);
                t += __shfl_xor_sync(0xffffffffu, t, 2);
                t += __shfl_xor_sync(0xffffffffu, t, 4);
                if (ok) {
                    // Q4_K keeps every aligned run of 8 in the order 0,2,1,3,4,6,5,7 (xh_index)
                    const int a1 = KIND == 3 ? 2 : 1, a2 = KIND == 3 ? 1 : 2;
                    const __half2 h01 = __halves2half2(h[0], h[a1]), h23 = __halves2half2(h[a2], h[3]);
                    const __half2 l01 = __halves2half2(l[0], l[a1]), l23 = __halves2half2(l[a2], l[3]);
                    *reinterpret_cast<uint2*>(hi + k) =
                        make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
                    *reinterpret_cast<uint2*>(lo + k) =
                        make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
                    if (f32) *reinterpret_cast<float4*>(f32 + k) = v;
                    if ((lane & 7) == 0) sx[k >> 5] = t;
                }
            } else if (ok) {
                *reinterpret_cast<float4*>(xs + xs_index<KIND>(k)) = v;
            }
        };
        float4 v[XQ_REG];
        double ss = 0.0;
#pragma unroll
        for (int j = 0; j < XQ_REG; ++j) {
            const int q = j * SG_CTHREADS + threadIdx.x;
            v[j] = (j < nrun && q < nq) ? ld_f4<CG>(x + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (RMS) ss += (double)v[j].x * v[j].x + (double)v[j].y * v[j].y + (double)v[j].z * v[j].z + (double)v[j].w * v[j].w;
        }
        float inv = 1.0f;
        if (RMS) {
            consumer_sum_d2<NC>(ss, extra, red);
            const double inv_d = 1.0 / sqrt(ss / (double)K + (double)eps);
            inv = isfinite(inv_d) ? (float)inv_d : 0.0f;
        } else if (EXTRA) {
            double z = 0.0;
            consumer_sum_d2<NC>(extra, z, red);
        }
#pragma unroll
        for (int j = 0; j < XQ_REG; ++j) {
            if (j < nrun) {
                const int q = j * SG_CTHREADS + threadIdx.x;
                const bool ok = q < nq;
                float4 o = v[j];
                if (RMS && ok) {
                    const float4 w4 = *reinterpret_cast<const float4*>(nw_s + 4 * q);
                    o = make_float4(o.x * inv * w4.x, o.y * inv * w4.y, o.z * inv * w4.z, o.w * inv * w4.w);
                }
                emit4(q, ok, o);
            }
        }
        consumer_sync<NC>();
        return extra;
    }
    // wide or unaligned rows: one value per thread and pass, raw values parked in shared
    // memory between the two passes of the normalisation
    const int nv = (K + SG_CTHREADS - 1) / SG_CTHREADS;
    auto emit = [&](int j, float val) {
        const int k = j * SG_CTHREADS + threadIdx.x;
        const bool ok = k < K;                       // uniform per warp: K % 32 == 0
        if (UsesMma<KIND>::value) {
            __half h, l;
            split_half(val, h, l);
            if (ok) {
                const int i = xh_index<KIND>(k);
                hi[i] = h;
                lo[i] = l;
                if (f32) f32[k] = val;
            }
            const float t = warp_sum(ok ? __half2float(h) + __half2float(l) : 0.0f);
            if (ok && lane == 0) sx[(j * SG_CTHREADS + warp * 32) >> 5] = t;
        } else if (ok) {
            xs[xs_index<KIND>(k)] = val;
        }
    };
    if (!RMS) {
        if (EXTRA) {
            double z = 0.0;
            consumer_sum_d2<NC>(extra, z, red);
        }
#pragma unroll 4
        for (int j = 0; j < nv; ++j) {
            const int k = j * SG_CTHREADS + threadIdx.x;
            emit(j, k < K ? ld_f1<CG>(x + k) : 0.0f);
        }
        consumer_sync<NC>();
        return extra;
    }
    double ss = 0.0;
    float* stash = UsesMma<KIND>::value ? f32 : xs;
    for (int j = 0; j < nv; ++j) {
        const int k = j * SG_CTHREADS + threadIdx.x;
        if (k < K) {
            const float val = ld_f1<CG>(x + k);
            stash[UsesMma<KIND>::value ? k : xs_index<KIND>(k)] = val;
            ss += (double)val * val;
        }
    }
    consumer_sum_d2<NC>(ss, extra, red);
    const double inv_d = 1.0 / sqrt(ss / (double)K + (double)eps);
    const float inv = isfinite(inv_d) ? (float)inv_d : 0.0f;
    for (int j = 0; j < nv; ++j) {
        const int k = j * SG_CTHREADS + threadIdx.x;
        emit(j, k < K ? stash[UsesMma<KIND>::value ? k : xs_index<KIND>(k)] * inv * nw_s[k] : 0.0f);
    }
    consumer_sync<NC>();
    return extra;
}

// `cnt` vectors of K floats (src + r * src_stride) into token rows 0..cnt-1 of xa in
// one pass: all loads in flight together, one barrier.  No normalisation.  Falls back
// to one stage_x per vector when the runs do not fit the registers.
// row_index (optional): row r is read from src + (row_index[r] / div) * src_stride (a gather).
// XQ: runs of four a thread may hold (cnt * K <= XQ * 4 * threads for the one-pass form).
template <int KIND, bool CG = false, int NC = SG_CONSUMERS, int XQ = XQ_REG>
__device__ __forceinline__ void stage_rows(const float* src, int64_t src_stride, const XAct& xa, int cnt,
                                           double* red, const int32_t* row_index = nullptr, int div = 1) {
    constexpr int SG_CTHREADS = NC * 32;
    const int K = xa.K, nq = K >> 2, total = cnt * nq;
    const int nrun = (total + SG_CTHREADS - 1) / SG_CTHREADS;
    auto row_of = [&](int r) -> int64_t { return row_index ? (int64_t)(row_index[r] / div) : (int64_t)r; };
    if (nrun > XQ || (reinterpret_cast<uintptr_t>(src) & 15) != 0 || (src_stride & 3) != 0) {
        for (int r = 0; r < cnt; ++r)
            stage_x<KIND, false, false, CG, NC>(src + row_of(r) * src_stride, nullptr, xa, r, 0.0f, red, 0.0);
        return;
    }
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)(K + XH_PAD);
    // i / nq by one multiplication (exact for i < 2^16 * ... : i <= XQ * threads, nq <= 2^14); the
    // gathered rows' numbers are worked out once, by cnt threads, into the reduction scratch
    const uint32_t nq_inv = 0xFFFFFFFFu / (uint32_t)nq + 1u;
    int* rix = reinterpret_cast<int*>(red);
    if (row_index) {
        if ((int)threadIdx.x < cnt) rix[threadIdx.x] = row_index[threadIdx.x] / div;
        consumer_sync<NC>();
    }
    float4 v[XQ];
#pragma unroll
    for (int j = 0; j < XQ; ++j) {
        const int i = j * SG_CTHREADS + threadIdx.x;
        const int r = (int)__umulhi((uint32_t)i, nq_inv), q = i - r * nq;
        const int64_t sr = row_index ? (int64_t)rix[min(r, cnt - 1)] : (int64_t)r;
        v[j] = (j < nrun && i < total) ? ld_f4<CG>(src + sr * src_stride + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < XQ; ++j) {
        if (j < nrun) {
            const int i = j * SG_CTHREADS + threadIdx.x;
            const bool ok = i < total;
            const int rr = (int)__umulhi((uint32_t)i, nq_inv);
            const int r = ok ? rr : 0, q = ok ? i - rr * nq : 0, k = q << 2;
            if (UsesMma<KIND>::value) {
                __half h[4], l[4];
                split_half(v[j].x, h[0], l[0]);
                split_half(v[j].y, h[1], l[1]);
                split_half(v[j].z, h[2], l[2]);
                split_half(v[j].w, h[3], l[3]);
                float t = 0.0f;
#pragma unroll
                for (int e = 0; e < 4; ++e) t += __half2float(h[e]) + __half2float(l[e]);
                if (!ok) t = 0.0f;
                t += __shfl_xor_sync(0xffffffffu, t, 1);
                t += __shfl_xor_sync(0xffffffffu, t, 2);
                t += __shfl_xor_sync(0xffffffffu, t, 4);
                if (ok) {
                    const int a1 = KIND == 3 ? 2 : 1, a2 = KIND == 3 ? 1 : 2;
                    const __half2 h01 = __halves2half2(h[0], h[a1]), h23 = __halves2half2(h[a2], h[3]);
                    const __half2 l01 = __halves2half2(l[0], l[a1]), l23 = __halves2half2(l[a2], l[3]);
                    *reinterpret_cast<uint2*>(xa.hi + r * row + k) =
                        make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
                    *reinterpret_cast<uint2*>(xa.lo + r * row + k) =
                        make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
                    if (xa.f32) *reinterpret_cast<float4*>(xa.f32 + (size_t)r * K + k) = v[j];
                    if ((lane & 7) == 0) xa.sumx[(size_t)r * (K >> 5) + (k >> 5)] = t;
                }
            } else if (ok) {
                *reinterpret_cast<float4*>(xa.xs + (size_t)r * xa.xs_tok + xs_index<KIND>(k)) = v[j];
            }
        }
    }
    consumer_sync<NC>();
}

// Dot products of a tile's rows with the staged activations of M tokens into
// red_pass[part][row][token] (part stride RED_PASSES * RED_PASS floats).
template <int KIND, int MT>
__device__ __forceinline__ void tile_compute(const uint8_t* tile, int64_t rb, int rows, int K, const XAct& xa,
                                             int tok0, int M, float* red_pass, int warp, int lane) {
    if (UsesMma<KIND>::value) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        XHalf xh = xa.half();
        xh.hi += (size_t)tok0 * xh.stride;
        xh.lo += (size_t)tok0 * xh.stride;
        xh.sumx += (size_t)tok0 * xh.nsub;
        xh.zero_row -= tok0;
        if (KIND == 3) tile_dot_q4k(tile, (int)rb, K, xh, M, warp, SG_CONSUMERS, lane, acc);
        else tile_dot_f16(tile, (int)rb, K, xh, M, warp, SG_CONSUMERS, lane, acc);
        float* o = red_pass + (size_t)warp * RED_PASSES * RED_PASS;
        const int gid = lane >> 2, c = 2 * (lane & 3);
        o[gid * RED_TOK + c] = acc[0];
        o[gid * RED_TOK + c + 1] = acc[1];
        o[(gid + 8) * RED_TOK + c] = acc[2];
        o[(gid + 8) * RED_TOK + c + 1] = acc[3];
    } else {
        for (int r = warp; r < rows; r += SG_CONSUMERS) {
            float acc[MT];
            row_dot_xs<KIND, MT>(tile + (int64_t)r * rb, xa.xs + (size_t)tok0 * xa.xs_tok, xa.xs_tok, M, K, lane, acc);
            if (lane < MT && lane < M) {
                float v = 0.0f;
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m == lane) v = acc[m];
                red_pass[r * RED_TOK + lane] = v;
            }
        }
    }
}

// Sum of the parts for element (row, token) of one pass.
template <int KIND>
__device__ __forceinline__ float red_value(const float* red_pass, int row, int tok) {
    if (!UsesMma<KIND>::value) return red_pass[row * RED_TOK + tok];
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < SG_CONSUMERS; ++w) v += red_pass[(size_t)w * RED_PASSES * RED_PASS + row * RED_TOK + tok];
    return v;
}
#endif

// ---- host helpers ---------------------------------------------------------------
template <typename Kern, typename Args>
static int launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, const Args& a) {
    if (a.dry) return B200_OK;          // shape check only: everything up to the launch has passed
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
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET_FULL));
    return B200_OK;
}

// Rows per tile.  Tensor-core kinds: always TILE_ROWS.  Others: about 8 KB, at most
// TILE_ROWS, a multiple of what keeps every tile (and sub-tile of `align_row_bytes`
// rows) 16-byte aligned.  Returns -1 when no such count exists.
static inline int pick_rows(int kind, int64_t bytes_per_row, int64_t align_a, int64_t align_b, int max_rows) {
    if (kind == 3 || kind == KIND_F16) return TILE_ROWS;
    int R = (int)std::max<int64_t>(1, 8192 / std::max<int64_t>(1, bytes_per_row));
    R = std::min(std::min(R, TILE_ROWS), std::max(1, max_rows));
    for (int r = R; r >= 1; --r)
        if ((r * align_a) % 16 == 0 && (r * align_b) % 16 == 0) return r;
    for (int r = R + 1; r <= TILE_ROWS; ++r)
        if ((r * align_a) % 16 == 0 && (r * align_b) % 16 == 0) return r;
    return -1;
}

// A bulk copy moves a multiple of 16 bytes: the last, shorter tile of `total_rows`
// rows must keep that property too (for each of the row sizes a tile carries).
static inline bool tail_tile_ok(int total_rows, int R, int64_t bytes_a, int64_t bytes_b = 0) {
    const int tail = total_rows % R;
    return (tail * bytes_a) % 16 == 0 && (tail * bytes_b) % 16 == 0;
}

// Stages of the ring: as many as fit the half-SM budget; when that leaves fewer than
// three (wide rows), the whole-SM budget is used instead.
static inline int pick_stages_in(size_t stage_bytes, size_t other_bytes, size_t budget) {
    int s = SG_MAX_STAGES;
    while (s > 1 && s * stage_bytes + other_bytes > budget) --s;
    return (s * stage_bytes + other_bytes <= budget) ? s : 0;
}
static inline int pick_stages(size_t stage_bytes, size_t other_bytes) {
    const int s = pick_stages_in(stage_bytes, other_bytes, SMEM_BUDGET);
    return s >= 3 ? s : std::max(s, pick_stages_in(stage_bytes, other_bytes, SMEM_BUDGET_FULL));
}

}  // namespace b200
