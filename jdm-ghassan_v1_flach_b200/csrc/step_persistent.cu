// Persistent decode-step kernel: the Mamba-2 and MoE phases of one token (batch 1) in
// a single cooperative launch, one CTA per SM.
//
// A token's step is a chain of ~200 dependent matrix-vector phases of 1-6 MB each.  As
// separate launches every phase pays a launch, a cold start of its weight stream and a
// drain.  Here all CTAs stay resident: the producer warp of each CTA walks the phase
// list ahead of the consumers and keeps its shared-memory ring full across phase
// boundaries (weights never depend on activations; only the routed experts' tiles wait
// for the router, and they are requested as soon as the router's logits exist, not when
// the phase that uses them begins), and the phases are separated by grid barriers - one
// arrival counter in global memory, release-add + acquire-spin with an iteration bound.
// Everything small and cold a phase needs (norm weights, per-head constants, the
// convolution taps and window of a tile's channels) is fetched ahead: the per-channel
// data rides in the tile's ring stage, the per-phase vectors are loaded while the
// preceding barrier is being waited for.  When a bound runs out the CTA raises the
// status word, the others see it and leave too, every producer drains its own copies,
// and the last CTA out zeroes the counters, so the call returns with an error and the
// next launch starts clean.
//
// Phase order and arithmetic: Generator::decode_step_logits / decode_mamba_layer
// (inference/generator.cpp:221-443, :456-617) and cpu::moe_forward_bias
// (core/moe_cpu.cpp:198-288); the dot-product engine, activation staging and exact-order
// router are those of the per-phase fused kernels (fused_common.cuh, fused_moe.cu).
#include "fused_common.cuh"
#include "persist.cuh"
#include "route.cuh"

namespace b200 {

#ifndef PS_CW_N
#define PS_CW_N 8
#endif
constexpr int PS_CW = PS_CW_N;        // consumer warps
constexpr int PS_CT = PS_CW * 32;     // consumer threads
constexpr int PS_THREADS = PS_CT + 32;
constexpr int PS_ROUTER_ROWS = 4;     // fp32 router rows per tile, one per consumer warp
constexpr int PS_UNIT = 8;            // rows of each of the two matrices packed into one 16-row tile
constexpr int PS_NS_MAX = 8;          // d_state / 32 state elements a lane keeps in registers
constexpr int PS_ROT = 53;            // CTA rotation per phase, spreads the light and heavy shares
constexpr unsigned PS_SMEM_SPIN = 1u << 24;      // iterations of a wait on a shared-memory word

// Control block in shared memory.
struct PCtl {
    uint64_t full[PS_MAX_STAGES], empty[PS_MAX_STAGES];
    double red_d[2 * PS_CW];
    double warp_sq[PS_CW];
    volatile int abort;        // a bounded wait of this CTA ran out (or the status word was seen raised)
    int snap;                  // abort as thread 0 saw it before a consumer barrier: one value for all threads
    volatile int route_gen;    // layer + 1 whose routing sits in r_idx / r_w [layer & 1]
    int r_idx[2][16];
    float r_w[2][16];
    float s_gate[PS_UNIT], s_xv[PS_UNIT];
};

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_volatile_s32(const int* p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ps_now() {
    return (unsigned long long)clock64();
}
// Phase timer: thread 0 of the traced CTA stamps slot `slot` of phase `oi`.
__device__ __forceinline__ void ps_stamp(const PArgs& a, int oi, int slot) {
    if (a.trace && threadIdx.x == 0 && (int)blockIdx.x == a.trace_cta)
        a.trace[(size_t)oi * PS_TRACE_SLOTS + slot] = ps_now();
}

// Bounded mbarrier wait.  The producer lane (WATCH_ABORT) also gives up when the CTA is
// aborting; the consumer warps do not look at that flag here: they all wait on the same
// barrier phase, so they pass or run out together and never split at a CTA barrier.
template <bool WATCH_ABORT>
__device__ __forceinline__ bool ps_mbar_wait(uint64_t* bar, uint32_t parity, PCtl* c, int* status) {
    for (uint32_t it = 0; it < MBAR_SPIN_LIMIT; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (WATCH_ABORT && (it & 15) == 15 && c->abort) return false;
    }
    atomicExch(status, 1);
    c->abort = 1;
    return false;
}

// Bounded wait of one thread for a global counter to reach `target`.
__device__ __forceinline__ bool ps_wait_counter(const PArgs& a, const unsigned int* ctr, unsigned target, PCtl* c) {
    for (unsigned it = 0; it < a.spin_limit; ++it) {
        if (ld_acquire_u32(ctr) >= target) return true;
        if ((it & 63) == 63 && (c->abort || ld_volatile_s32(a.status) != 0)) break;
    }
    atomicExch(a.status, 1);
    c->abort = 1;
    return false;
}

// ---- per-tile dot products (one token) ---------------------------------------------
// red: [PS_CW][16] floats.  Tensor-core kinds: warp `w` leaves its share of K for the
// tile's 16 rows in red[w][row]; scalar kinds: the warp that owns a row leaves the whole
// sum in red[0][row].
template <int KIND>
__device__ __forceinline__ void ps_tile_acc(const uint8_t* tile, int rb, int K, const XAct& xa, int tok, int slice,
                                         int lane, float (&acc)[4]) {
    XHalf xh = xa.half();
    xh.hi += (size_t)tok * xh.stride;
    xh.lo += (size_t)tok * xh.stride;
    xh.sumx += (size_t)tok * xh.nsub;
    xh.zero_row -= tok;
    // one slice: 64 weights of every row (Q4_K) or 32 (fp16)
    if (KIND == 3) tile_dot_q4k(tile, rb, K, xh, 1, slice, 1 << 28, lane, acc);
    else tile_dot_f16(tile, rb, K, xh, 1, slice, 1 << 28, lane, acc);
}
__device__ __forceinline__ void ps_acc_store(const float (&acc)[4], float* red, int warp, int lane) {
    if ((lane & 3) == 0) {
        red[warp * 16 + (lane >> 2)] = acc[0];
        red[warp * 16 + (lane >> 2) + 8] = acc[2];
    }
}
template <int KIND>
__device__ __forceinline__ float ps_red_val(const float* red, int row) {
    if (!UsesMma<KIND>::value) return red[row];
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < PS_CW; ++w) v += red[w * 16 + row];
    return v;
}

// Activation staging for the kernel's one token: `cnt` vectors of K floats (src + r *
// stride; written by other CTAs, hence L2 loads) into rows 0..cnt-1 of xa - fp16 hi + lo
// parts and 32-wide sums for the tensor-core kinds, fp32 unit-major for the scalar kinds
// (the layouts of fused_common.cuh / mma_tile.cuh).  rms: v <- v * inv_rms * nw in the
// reference's operand order (core/math_cpu.cpp:299-316, double sum of squares); reduce:
// `extra` is summed over the consumer threads in the same reduction and returned.  One
// shared, compact copy: K % 32 == 0, cnt * K <= 16 * PS_CT, 16-byte aligned rows.
constexpr int PS_XQ = 4;
// Every phase calls this one copy (arguments by value: nothing of the caller's goes
// through local memory).
template <int KIND>
__device__ __noinline__ double ps_stage_impl(const float* src, int64_t stride, int cnt, const float* nw, __half* xa_hi,
                                             __half* xa_lo, float* xa_sumx, float* xa_f32, float* xa_xs, int xa_xs_tok,
                                             int K, float eps, double* red, double extra, bool rms, bool reduce) {
    struct { __half *hi, *lo; float *sumx, *f32, *xs; int xs_tok; } xa = {xa_hi, xa_lo, xa_sumx, xa_f32, xa_xs, xa_xs_tok};
    const int nq = K >> 2, total = cnt * nq;
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)(K + XH_PAD);
    float4 v[PS_XQ];
    int rr[PS_XQ], qq[PS_XQ];
    double ss = 0.0;
#pragma unroll
    for (int j = 0; j < PS_XQ; ++j) {
        const int i = j * PS_CT + (int)threadIdx.x;
        const bool ok = i < total;
        const int r = (ok && cnt > 1) ? i / nq : 0;
        rr[j] = r;
        qq[j] = ok ? i - r * nq : 0;
        v[j] = ok ? __ldcg(reinterpret_cast<const float4*>(src + r * stride + 4 * qq[j])) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (rms) ss += (double)v[j].x * v[j].x + (double)v[j].y * v[j].y + (double)v[j].z * v[j].z + (double)v[j].w * v[j].w;
    }
    float inv = 1.0f;
    if (rms || reduce) {
        consumer_sum_d2<PS_CW>(ss, extra, red);
        if (rms) {
            const double inv_d = 1.0 / sqrt(ss / (double)K + (double)eps);
            inv = isfinite(inv_d) ? (float)inv_d : 0.0f;
        }
    }
#pragma unroll
    for (int j = 0; j < PS_XQ; ++j) {
        if (j * PS_CT < total) {                       // uniform: every lane takes part in the shuffles
            const int i = j * PS_CT + (int)threadIdx.x;
            const bool ok = i < total;
            const int r = rr[j], q = qq[j], k = q << 2;
            float4 o = v[j];
            if (rms && ok) {
                const float4 w4 = *reinterpret_cast<const float4*>(nw + k);
                o = make_float4(o.x * inv * w4.x, o.y * inv * w4.y, o.z * inv * w4.z, o.w * inv * w4.w);
            }
            if (UsesMma<KIND>::value) {
                __half h[4], l[4];
                split_half(o.x, h[0], l[0]);
                split_half(o.y, h[1], l[1]);
                split_half(o.z, h[2], l[2]);
                split_half(o.w, h[3], l[3]);
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
                    *reinterpret_cast<uint2*>(xa.hi + r * row + k) =
                        make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
                    *reinterpret_cast<uint2*>(xa.lo + r * row + k) =
                        make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
                    if (xa.f32) *reinterpret_cast<float4*>(xa.f32 + (size_t)r * K + k) = o;
                    if ((lane & 7) == 0) xa.sumx[(size_t)r * (K >> 5) + (k >> 5)] = t;
                }
            } else if (ok) {
                *reinterpret_cast<float4*>(xa.xs + (size_t)r * xa.xs_tok + xs_index<KIND>(k)) = o;
            }
        }
    }
    consumer_sync<PS_CW>();
    return extra;
}
template <int KIND>
__device__ __forceinline__ double ps_stage(const float* src, int64_t stride, int cnt, const float* nw, const XAct& xa,
                                           float eps, double* red, double extra, bool rms, bool reduce) {
    return ps_stage_impl<KIND>(src, stride, cnt, nw, xa.hi, xa.lo, xa.sumx, xa.f32, xa.xs, xa.xs_tok, xa.K, eps, red, extra,
                               rms, reduce);
}

// One causal-convolution step of a channel: window of raw inputs, oldest first, unfused
// operations in the reference's order (inference/generator.cpp:520-560).  taps, window
// and bias were fetched with the tile; the shifted window goes back to global memory.
// Returns the pre-activation sum.
__device__ __forceinline__ float ps_conv_step(int k, const float (&wp)[8], const float (&sp)[8], float bias,
                                              float* sp_out, float v) {
    const int win = k - 1;
    float t = bias;
    float wl = wp[0];
#pragma unroll
    for (int j = 0; j < 7; ++j) {
        if (j < win) {
            t = __fadd_rn(t, __fmul_rn(wp[j], sp[j]));
            if (j > 0) sp_out[j - 1] = sp[j];
            wl = wp[j + 1];
        }
    }
    t = __fadd_rn(t, __fmul_rn(wl, v));
    if (win > 0) sp_out[win - 1] = v;
    return t;
}

// Position in the ring: stage index, phase parity of its barriers, parity of the tile
// count (selects the reduction buffer).
struct PRingPos {
    unsigned st = 0, ph = 0, odd = 0;
    __device__ __forceinline__ void advance(int n_stages) {
        odd ^= 1u;
        if (++st == (unsigned)n_stages) { st = 0; ph ^= 1u; }
    }
};

struct PView {          // this CTA's shared memory, carved by the host's plan
    uint8_t* stages;
    XAct xa1, xa2, xa3;
    uint8_t* xa2_base;
    float *nw, *gs, *red, *r_p, *r_sel, *bcd, *hp, *rbias;
    const POp* ops;         // [op_end - op_begin]
    const PLayer* layers;   // [n_layers]
    PCtl* c;
};

// Consumer side of the ring: wait for the tile at `rp` (all consumer warps call this).
__device__ __forceinline__ const uint8_t* ps_take(const PArgs& a, const PView& s, const PRingPos& rp, bool& ok) {
    ok = ps_mbar_wait<false>(&s.c->full[rp.st], rp.ph, s.c, a.status);
    return s.stages + (size_t)rp.st * a.stage_bytes;
}

// Dot products of the <= 16 rows of a tile with the staged activations `tok` of xa, the
// stage handed back to the producer, the warps' partial sums added: returns the value of
// row threadIdx.x in threads 0..15 (0 elsewhere).  Ends behind a consumer barrier.
// ntok > 1: the tile holds ntok sub-tiles `sub` bytes apart, sub-tile k is multiplied with
// token row k of xa and the results are mixed with the weights wk (the routed experts'
// down projections); ntok == 1, wk == nullptr: the plain product.
template <int KIND>
__device__ __forceinline__ float ps_rows(const uint8_t* ts, int rb, int nrows, int K, const XAct& xa, int ntok, int sub,
                                      const float* wk, float* red, uint64_t* empty) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (UsesMma<KIND>::value) {
        // units (token k, slice g of K) dealt round-robin to the warps
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const int slices = KIND == 3 ? K >> 6 : K >> 5, total = ntok * slices;
        for (int q = warp; q < total; q += PS_CW) {
            const int k = ntok > 1 ? q / slices : 0, g = q - k * slices;
            float t[4] = {0.f, 0.f, 0.f, 0.f};
            ps_tile_acc<KIND>(ts + (size_t)k * sub, rb, K, xa, k, g, lane, t);
            const float w = wk ? wk[k] : 1.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] += w * t[j];
        }
        ps_acc_store(acc, red, warp, lane);
    } else {
        for (int r = warp; r < nrows; r += PS_CW) {
            float acc = 0.0f, t[1];
            for (int k = 0; k < ntok; ++k) {
                row_dot_xs<KIND, 1>(ts + (size_t)k * sub + (int64_t)r * rb, xa.xs + (size_t)k * xa.xs_tok, xa.xs_tok, 1, K,
                                    lane, t);
                acc = __fadd_rn(acc, __fmul_rn(wk ? wk[k] : 1.0f, t[0]));
            }
            if (lane == 0) red[r] = acc;
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty);
    consumer_sync<PS_CW>();
    return threadIdx.x < 16 ? ps_red_val<KIND>(red, threadIdx.x) : 0.0f;
}
__device__ __forceinline__ float ps_silu(float v) { return silu_acc(v); }

// Tiles of a phase owned by this CTA: t = v, v + grid, ...
__device__ __forceinline__ int ps_rot(int op_index) { return (int)((blockIdx.x + (unsigned)op_index * PS_ROT) % gridDim.x); }
__device__ __forceinline__ int ps_mamba_bc_tiles(const PArgs& a) { return (2 * a.d_state + a.n_heads + 15) / 16; }

// Layout of a Mamba in_proj tile's ring stage behind the 16 weight rows.
//   head unit:  [8 state rows][taps 8 x k][window 8 x (k-1)][bias 8][norm weight 8]
//   B/C tile:   [taps 16 x k][window 16 x (k-1)][bias 16]
struct PTileExtra {
    int state, taps, window, bias, norm;
};
__device__ __forceinline__ PTileExtra ps_unit_extra(const PArgs& a, int rb) {
    PTileExtra e;
    e.state = 16 * rb;
    e.taps = e.state + PS_UNIT * a.d_state * 4;
    e.window = e.taps + PS_UNIT * a.dconv * 4;
    e.bias = e.window + PS_UNIT * (a.dconv - 1) * 4;
    e.norm = e.bias + PS_UNIT * 4;
    return e;
}
__device__ __forceinline__ PTileExtra ps_bc_extra(const PArgs& a, int rb) {
    PTileExtra e;
    e.state = 0;
    e.taps = 16 * rb;
    e.window = e.taps + 16 * a.dconv * 4;
    e.bias = e.window + 16 * (a.dconv - 1) * 4;
    e.norm = 0;
    return e;
}

// ---- consumer side of each phase ---------------------------------------------------
template <int KIND>
struct PConsumer {
    const PArgs& a;
    PView& s;
    int warp, lane;
    PRingPos rp;                 // next tile to take from the ring
    unsigned mamba_seen = 0;     // POP_MAMBA_A phases finished in this launch
    int cur_op = 0;              // phase index, for the phase timers

    long long wait_cyc = 0, rows_cyc = 0;    // phase timers: cycles spent waiting for tiles / in the dot routine
    __device__ __forceinline__ const uint8_t* take(bool& ok) {
        const long long t0 = a.trace ? clock64() : 0;
        const uint8_t* p = ps_take(a, s, rp, ok);
        if (a.trace) wait_cyc += clock64() - t0;
        return p;
    }
    __device__ __forceinline__ void give() {
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.c->empty[rp.st]);
        rp.advance(a.n_stages);
    }
    // dot products of a <= 16-row tile, stage handed back, partials reduced: the value of
    // row threadIdx.x in threads 0..15 (one shared routine for every phase)
    __device__ __forceinline__ float rows(const uint8_t* ts, int rb, int nrows, int K, const XAct& xa, int ntok = 1,
                                          int sub = 0, const float* wk = nullptr) {
        const long long t0 = a.trace ? clock64() : 0;
        const float v = ps_rows<KIND>(ts, rb, nrows, K, xa, ntok, sub, wk, s.red + rp.odd * (PS_CW * 16), &s.c->empty[rp.st]);
        if (a.trace) rows_cyc += clock64() - t0;
        rp.advance(a.n_stages);
        return v;
    }
    // SwiGLU of a tile that packs 8 gate rows (threads 0-7 hold them) over 8 up rows
    // (threads 8-15): silu(g) * u in threads 0-7
    __device__ __forceinline__ float swiglu8(float v) {
        const float u = __shfl_down_sync(0xffffffffu, v, PS_UNIT);
        return ps_silu(v) * u;
    }

    // Loads that do not depend on the phases before `op`: issued by the warps that do not
    // run the grid barrier while it is being waited for (or by all before the first phase).
    __device__ __forceinline__ void prefetch(const POp op, int first_thread) {
        if (op.op != POP_MAMBA_A && op.op != POP_MOE_C) return;
        const PLayer& L = s.layers[op.layer];
        const int nt = PS_CT - first_thread, t0 = (int)threadIdx.x - first_thread;
        if (t0 < 0) return;
        const float* nw = op.op == POP_MAMBA_A ? L.attn_norm : L.ffn_norm;
        for (int k = t0 * 4; k < a.d; k += nt * 4)
            *reinterpret_cast<float4*>(s.nw + k) = __ldg(reinterpret_cast<const float4*>(nw + k));
        if (op.op == POP_MAMBA_A)
            for (int h = t0; h < a.n_heads; h += nt) {
                s.hp[h] = L.dt_bias[h];
                s.hp[a.n_heads + h] = L.a_log[h];
                s.hp[2 * a.n_heads + h] = L.D[h];
            }
    }

    __device__ bool embed() {
        const int64_t tok = a.tok[0];
        for (int i = blockIdx.x * PS_CT + threadIdx.x; i < a.d; i += gridDim.x * PS_CT) {
            float v = half_bits_to_float(a.embed[tok * a.d + i]);
            if (a.emb_mult != 1.0f) v *= a.emb_mult;
            a.x[i] = v;
        }
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            const int p = a.len[0];
            a.pos[0] = p;
            a.len[0] = p + 1;
        }
        return true;
    }

    // taps, window and bias of row `i` of a tile whose extras sit at `e`
    __device__ __forceinline__ void conv_operands(const uint8_t* ts, const PTileExtra& e, int i, bool has_bias,
                                                  float (&tp)[8], float (&sw)[8], float& bias) {
        const int k = a.dconv, win = k - 1;
        const float* wp = reinterpret_cast<const float*>(ts + e.taps) + i * k;
        const float* sp = reinterpret_cast<const float*>(ts + e.window) + i * win;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            tp[j] = j < k ? wp[j] : 0.0f;
            sw[j] = j < win ? sp[j] : 0.0f;
        }
        bias = has_bias ? reinterpret_cast<const float*>(ts + e.bias)[i] : 0.0f;
    }

    __device__ bool mamba_a(const PLayer& L, int op_index) {
        const int d = a.d, ds = a.d_state, nh = a.n_heads, k = a.dconv, win = k - 1;
        const int rb = (int)row_bytes_of(KIND, d);
        ps_stage<KIND>(a.x, 0, 1, s.nw, s.xa1, a.eps, s.c->red_d, 0.0, true, false);
        ps_stamp(a, cur_op, 1);
        const int nbc = ps_mamba_bc_tiles(a), nconv_tiles = (2 * ds) / 16, ntiles = nbc + a.d_inner / PS_UNIT;
        const int ns = ds >> 5;                              // state elements per lane
        bool bc_loaded = false;
        double sq = 0.0;
        for (int t = ps_rot(op_index); t < ntiles; t += gridDim.x) {
            bool ok;
            const uint8_t* ts = take(ok);
            if (!ok) return false;
            if (t < nbc) {
                // rows of B, C (convolved below) or dt
                const int r0 = 2 * a.d_inner + t * 16, nrows = min(16, a.proj - r0);
                const bool conv_tile = t < nconv_tiles;
                float tp[8], sw[8], bias = 0.0f;
                if (conv_tile && threadIdx.x < 16) conv_operands(ts, ps_bc_extra(a, rb), threadIdx.x, L.conv_b != nullptr, tp, sw, bias);
                const float wv = rows(ts, rb, nrows, d, s.xa1);
                if ((int)threadIdx.x < nrows) {
                    if (conv_tile) {
                        const int c = r0 - a.d_inner + (int)threadIdx.x;       // convolution channel
                        const float pre = ps_conv_step(k, tp, sw, bias, L.conv_state + (int64_t)c * win, wv);
                        a.bcd[c - a.d_inner] = ps_silu(pre);
                    } else {
                        a.bcd[2 * ds + (r0 + (int)threadIdx.x - a.d_inner - a.conv_dim)] = wv;
                    }
                    __threadfence();
                }
                if (warp == 0) {
                    __syncwarp();
                    if (lane == 0) {
                        __threadfence();
                        atomicAdd(a.bc_flag, 1u);
                    }
                }
            } else {
                // 8 gate rows + the 8 matching x rows + their 8 state rows
                const int u = t - nbc;
                const PTileExtra e = ps_unit_extra(a, rb);
                float sv[PS_NS_MAX];
                float nwr = 0.0f;
                if (warp < PS_UNIT) {
                    nwr = reinterpret_cast<const float*>(ts + e.norm)[warp];
                    const float* st = reinterpret_cast<const float*>(ts + e.state) + (size_t)warp * ds;
                    if (ds == 128) {
                        const float4 q4 = *reinterpret_cast<const float4*>(st + lane * 4);
                        sv[0] = q4.x; sv[1] = q4.y; sv[2] = q4.z; sv[3] = q4.w;
                    } else {
#pragma unroll
                        for (int j = 0; j < PS_NS_MAX; ++j)
                            if (j < ns) sv[j] = st[j * 32 + lane];
                    }
                }
                float tp[8], sw[8], bias = 0.0f;
                if (threadIdx.x >= PS_UNIT && threadIdx.x < 2 * PS_UNIT)
                    conv_operands(ts, e, threadIdx.x - PS_UNIT, L.conv_b != nullptr, tp, sw, bias);
                const float v = rows(ts, rb, 16, d, s.xa1);
                if (threadIdx.x < PS_UNIT) {
                    s.c->s_gate[threadIdx.x] = v;
                } else if (threadIdx.x < 2 * PS_UNIT) {
                    const int c = u * PS_UNIT + threadIdx.x - PS_UNIT;
                    s.c->s_xv[threadIdx.x - PS_UNIT] = ps_silu(ps_conv_step(k, tp, sw, bias, L.conv_state + (int64_t)c * win, v));
                }
                if (!bc_loaded && threadIdx.x == 0) {
                    // B, C and dt of this token come from other CTAs' tiles of this phase
                    ps_wait_counter(a, a.bc_flag, (mamba_seen + 1) * (unsigned)nbc, s.c);
                    s.c->snap = s.c->abort;
                }
                consumer_sync<PS_CW>();
                if (!bc_loaded && s.c->snap) return false;
                if (!bc_loaded) {
                    for (int j = threadIdx.x; j < 2 * ds + nh; j += PS_CT) s.bcd[j] = __ldcg(a.bcd + j);
                    consumer_sync<PS_CW>();
                    bc_loaded = true;
                }
                // state update of row r (one warp per row): core of decode_mamba_layer,
                // inference/generator.cpp:562-600
                if (warp >= PS_UNIT) continue;
                const int r = u * PS_UNIT + warp, h = r / a.d_head;
                const float xv = s.c->s_xv[warp], gt = s.c->s_gate[warp];
                const float uu = s.bcd[2 * ds + h] + s.hp[h];
                const float dt = (uu > 20.0f) ? uu : log1pf(expf(uu));
                const float A = -expf(s.hp[nh + h]);
                const float dA = expf(__fmul_rn(A, dt));
                const float* Bv = s.bcd;
                const float* Cv = s.bcd + ds;
                float* sg = L.ssm_state + (int64_t)r * ds;
                float acc = 0.0f;
                if (ds == 128) {
                    const float4 b4 = *reinterpret_cast<const float4*>(Bv + lane * 4);
                    const float4 c4 = *reinterpret_cast<const float4*>(Cv + lane * 4);
                    float4 o;
                    o.x = __fadd_rn(__fmul_rn(dA, sv[0]), __fmul_rn(__fmul_rn(dt, b4.x), xv));
                    o.y = __fadd_rn(__fmul_rn(dA, sv[1]), __fmul_rn(__fmul_rn(dt, b4.y), xv));
                    o.z = __fadd_rn(__fmul_rn(dA, sv[2]), __fmul_rn(__fmul_rn(dt, b4.z), xv));
                    o.w = __fadd_rn(__fmul_rn(dA, sv[3]), __fmul_rn(__fmul_rn(dt, b4.w), xv));
                    *reinterpret_cast<float4*>(sg + lane * 4) = o;
                    acc = c4.x * o.x + c4.y * o.y + c4.z * o.z + c4.w * o.w;
                } else {
#pragma unroll
                    for (int j = 0; j < PS_NS_MAX; ++j) {
                        if (j < ns) {
                            const int el = j * 32 + lane;
                            const float sn = __fadd_rn(__fmul_rn(dA, sv[j]), __fmul_rn(__fmul_rn(dt, Bv[el]), xv));
                            sg[el] = sn;
                            acc += Cv[el] * sn;
                        }
                    }
                }
                acc = warp_sum(acc);
                if (lane == 0) {
                    const float y = acc + s.hp[2 * nh + h] * xv;
                    const float v = y * ps_silu(gt);
                    a.u[r] = v * nwr;
                    sq += (double)v * v;
                }
            }
        }
        if (lane == 0) s.c->warp_sq[warp] = sq;
        consumer_sync<PS_CW>();
        if (threadIdx.x == 0) {
            double t = 0.0;
            for (int w = 0; w < PS_CW; ++w) t += s.c->warp_sq[w];
            a.partials[blockIdx.x] = t;
        }
        ++mamba_seen;
        return true;
    }

    __device__ bool mamba_b(const PLayer& L, int op_index) {
        const int K = a.d_inner;
        const int rb = (int)row_bytes_of(KIND, K);
        xact_carve<KIND>(s.xa2, s.xa2_base, K, 1, false);
        xact_zero_row<KIND, PS_CW>(s.xa2);
        double t = 0.0;
        for (int i = threadIdx.x; i < (int)gridDim.x; i += PS_CT) t += __ldcg(a.partials + i);
        t = ps_stage<KIND>(a.u, 0, 1, nullptr, s.xa2, 0.0f, s.c->red_d, t, false, true) / (double)K;
        const float in_scale = 1.0f / sqrtf((float)t + a.eps);
        ps_stamp(a, cur_op, 1);
        const int ntiles = (a.d + 15) / 16;
        for (int tl = ps_rot(op_index); tl < ntiles; tl += gridDim.x) {
            const int r0 = tl * 16, nrows = min(16, a.d - r0);
            const bool owner = (int)threadIdx.x < nrows;
            float* dst = a.x + r0 + threadIdx.x;
            const float pre = owner ? __ldcg(dst) : 0.0f;
            bool ok;
            const uint8_t* ts = take(ok);
            if (!ok) return false;
            const float v = rows(ts, rb, nrows, K, s.xa2);
            if (owner) *dst = pre + v * in_scale * a.res_mult;
        }
        return true;
    }

    // Router logit of one expert in the reference's exact fp32 order (core/moe_cpu.cpp:76-83).
    __device__ __forceinline__ float router_logit_ps(const float* wrow, float* gs, int d) {
        const int groups = d >> 2;
        const XAct& xa = s.xa1;
        const float* xf = UsesMma<KIND>::value ? xa.f32 : xa.xs;
        for (int g = lane; g < groups; g += 32) {
            const float4 b = *reinterpret_cast<const float4*>(wrow + 4 * g);
            const int xi = UsesMma<KIND>::value ? 4 * g : xs_index<KIND>(4 * g);
            const float4 x4 = *reinterpret_cast<const float4*>(xf + xi);
            float t = __fadd_rn(__fmul_rn(x4.x, b.x), __fmul_rn(x4.y, b.y));
            t = __fadd_rn(t, __fmul_rn(x4.z, b.z));
            t = __fadd_rn(t, __fmul_rn(x4.w, b.w));
            gs[g] = t;
        }
        __syncwarp();
        float chain = 0.0f;
        if (lane == 0) {
#pragma unroll 8
            for (int g = 0; g < groups; ++g) chain = __fadd_rn(chain, gs[g]);
        }
        __syncwarp();
        return chain;
    }

    __device__ bool moe_c(const PLayer& L, int op_index) {
        const int d = a.d;
        const int rb = (int)row_bytes_of(KIND, d);
        ps_stage<KIND>(a.x, 0, 1, s.nw, s.xa1, a.eps, s.c->red_d, 0.0, true, false);
        ps_stamp(a, cur_op, 1);
        const int n_router = (a.ne + PS_ROUTER_ROWS - 1) / PS_ROUTER_ROWS;
        const int ntiles = n_router + (L.has_shared ? a.SH / PS_UNIT : 0);
        for (int t = ps_rot(op_index); t < ntiles; t += gridDim.x) {
            bool ok;
            const uint8_t* ts = take(ok);
            if (!ok) return false;
            if (t < n_router) {
                const int e = t * PS_ROUTER_ROWS + warp;
                if (warp < PS_ROUTER_ROWS && e < a.ne) {
                    const float* wrow = reinterpret_cast<const float*>(ts) + (int64_t)warp * d;
                    const float lg = router_logit_ps(wrow, s.gs + warp * (d >> 2), d);
                    if (lane == 0) {
                        a.logits[e] = lg;
                        __threadfence();
                        atomicAdd(a.rt_flag, 1u);      // one count per expert: the producers route when all are in
                    }
                }
                give();
            } else {
                const int r0 = (t - n_router) * PS_UNIT;
                const float v = rows(ts, rb, 16, d, s.xa1);
                if (warp == 0) {
                    const float o = swiglu8(v);
                    if (lane < PS_UNIT) a.sh_act[r0 + lane] = o;
                }
            }
        }
        return true;
    }

    __device__ bool moe_d(const PLayer& L, int op_index) {
        const int d = a.d;
        const int rb_d = (int)row_bytes_of(KIND, d);
        const int n_sd = L.has_shared ? (d + 15) / 16 : 0;
        const int per_slot = a.E / PS_UNIT;
        const int ntiles = n_sd + a.K * per_slot;
        int rb_sh = 0;
        if (L.has_shared) {
            rb_sh = (int)row_bytes_of(KIND, a.SH);
            xact_carve<KIND>(s.xa2, s.xa2_base, a.SH, 1, false);
            xact_zero_row<KIND, PS_CW>(s.xa2);
            ps_stage<KIND>(a.sh_act, 0, 1, nullptr, s.xa2, 0.0f, s.c->red_d, 0.0, false, false);
        }
        ps_stamp(a, cur_op, 1);
        for (int t = ps_rot(op_index); t < ntiles; t += gridDim.x) {
            bool ok;
            const uint8_t* ts = take(ok);
            if (!ok) return false;
            if (t < n_sd) {
                const int r0 = t * 16, nrows = min(16, d - r0);
                const float v = rows(ts, rb_sh, nrows, a.SH, s.xa2);
                if ((int)threadIdx.x < nrows) a.sh_out[r0 + threadIdx.x] = v;
            } else {
                const int i = t - n_sd, k = i / per_slot, r0 = (i % per_slot) * PS_UNIT;
                const float v = rows(ts, rb_d, 16, d, s.xa1);
                if (warp == 0) {
                    const float o = swiglu8(v);
                    if (lane < PS_UNIT) a.act[(int64_t)k * a.E + r0 + lane] = o;
                }
            }
        }
        return true;
    }

    __device__ bool moe_e(const PLayer& L, int layer, int op_index) {
        const int d = a.d, E = a.E, K = a.K;
        const int rb = (int)row_bytes_of(KIND, E);
        const int sub = 16 * rb;
        ps_stage<KIND>(a.act, E, K, nullptr, s.xa3, 0.0f, s.c->red_d, 0.0, false, false);
        // mixture weights: left in shared memory by this CTA's producer warp
        if (threadIdx.x == 0) {
            bool got = false;
            for (unsigned it = 0; it < PS_SMEM_SPIN; ++it) {
                if (s.c->route_gen == layer + 1) { got = true; break; }
                if (s.c->abort) break;
            }
            if (!got) {
                if (!s.c->abort) atomicExch(a.status, 1);
                s.c->abort = 1;
            }
            s.c->snap = s.c->abort;
        }
        consumer_sync<PS_CW>();
        if (s.c->snap) return false;
        const float* wk = s.c->r_w[layer & 1];
        ps_stamp(a, cur_op, 1);
        const int ntiles = (d + 15) / 16;
        for (int tl = ps_rot(op_index); tl < ntiles; tl += gridDim.x) {
            const int r0 = tl * 16, nrows = min(16, d - r0);
            const bool owner = (int)threadIdx.x < nrows;
            float* dst = a.x + r0 + threadIdx.x;
            float pre = 0.0f, sho = 0.0f;
            if (owner) {
                pre = __ldcg(dst);
                if (L.has_shared) sho = __ldcg(a.sh_out + r0 + threadIdx.x);
            }
            bool ok;
            const uint8_t* ts = take(ok);
            if (!ok) return false;
            const float v = rows(ts, rb, nrows, E, s.xa3, K, sub, wk);
            if (owner) *dst = pre + (sho + v) * a.res_mult;
        }
        return true;
    }

    // Grid barrier of the consumer threads (barriers passed so far: nbar).  Thread 0
    // arrives and waits; the other warps meanwhile fetch what the next phase needs that
    // no earlier phase produces.
    __device__ __forceinline__ bool grid_sync(unsigned& nbar, const POp next) {
        __threadfence();
        consumer_sync<PS_CW>();
        if (threadIdx.x == 0) {
            if ((int)blockIdx.x == a.skip_cta && nbar == 0) {
                s.c->abort = 1;                                   // test hook: never arrives
            } else {
                const unsigned long long target = (unsigned long long)(nbar + 1) * gridDim.x;
                atomicAdd(a.bar, 1ULL);
                bool ok = false;
                for (unsigned it = 0; it < a.spin_limit; ++it) {
                    if (ld_acquire_u64(a.bar) >= target) { ok = true; break; }
                    if ((it & 63) == 63 && ld_volatile_s32(a.status) != 0) break;
                }
                if (!ok) {
                    atomicExch(a.status, 1);
                    s.c->abort = 1;
                }
            }
            s.c->snap = s.c->abort;
        }
        prefetch(next, 32);
        consumer_sync<PS_CW>();
        ++nbar;
        return s.c->snap == 0;
    }
};

// ---- producer side -----------------------------------------------------------------
// Routing of the kernel's one token by one warp: softmax over the ne logits, K rounds of
// arg-max, renormalised mixture weights - the arithmetic of route_finish_warp (route.cuh;
// core/math_cpu.cpp:546-558, core/moe_cpu.cpp:85-98, 233-254) operation for operation,
// including the sequential e = 0, 1, ... order of the softmax denominator.  Written as
// small rolled loops over shared memory: this runs once per layer on cold instructions,
// and on this part an instruction fetched from L2 costs tens of cycles, so the size of
// the code, not its operation count, is what the routed experts' weights wait for.
// s_p, s_sel: ne floats each.
__device__ __noinline__ void ps_route_warp(const float* logits, const float* bias, int ne, int K, float* s_p,
                                           float* s_sel, int* s_idx, float* s_w, int lane) {
    float mx = -INFINITY;
#pragma unroll 1
    for (int e = lane; e < ne; e += 32) {
        const float v = __ldcg(logits + e);
        s_sel[e] = v;
        mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
#pragma unroll 1
    for (int e = lane; e < ne; e += 32) s_p[e] = (float)exp((double)__fsub_rn(s_sel[e], mx));
    __syncwarp();
    // denominator in the order e = 0, 1, 2, ... (every lane adds the same sequence)
    float sum = 0.0f;
#pragma unroll 4
    for (int e = 0; e < ne; ++e) sum = __fadd_rn(sum, s_p[e]);
    const float inv = (sum > 1e-12f) ? __fdiv_rn(1.0f, sum) : 0.0f;
    __syncwarp();
#pragma unroll 1
    for (int e = lane; e < ne; e += 32) {
        const float pr = __fmul_rn(s_p[e], inv);
        s_p[e] = pr;
        s_sel[e] = bias ? __fadd_rn(pr, bias[e]) : pr;
    }
    __syncwarp();
#pragma unroll 1
    for (int k = 0; k < K; ++k) {
        float bv = -1e30f;
        int bi = -1;
#pragma unroll 1
        for (int e = lane; e < ne; e += 32) {
            const float v = s_sel[e];
            if (v > bv) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        const int pick = bi < 0 ? 0 : bi;
        if (lane == 0) {
            s_idx[k] = pick;
            s_w[k] = s_p[pick];
            s_sel[pick] = -INFINITY;          // taken: never above the -1e30 floor again
        }
        __syncwarp();
    }
    if (lane == 0) {
        float sum_w = 0.0f;
#pragma unroll 1
        for (int k = 0; k < K; ++k) sum_w = __fadd_rn(sum_w, s_w[k]);
        const bool renorm = sum_w > 1e-8f;
        const float f = renorm ? __fdiv_rn(1.0f, sum_w) : __fdiv_rn(1.0f, (float)K);
#pragma unroll 1
        for (int k = 0; k < K; ++k) s_w[k] = renorm ? __fmul_rn(s_w[k], f) : f;
    }
    __syncwarp();
}

__device__ __forceinline__ bool ps_slot(const PArgs& a, const PView& s, const PRingPos& rp, unsigned seq, uint8_t*& dst,
                                     uint64_t*& full) {
    if (seq >= (unsigned)a.n_stages && !ps_mbar_wait<true>(&s.c->empty[rp.st], rp.ph ^ 1u, s.c, a.status)) return false;
    dst = s.stages + (size_t)rp.st * a.stage_bytes;
    full = &s.c->full[rp.st];
    return true;
}

template <int KIND>
struct PProducer {
    const PArgs& a;
    PView& s;
    int lane;
    PRingPos rp;             // next stage to fill
    unsigned seq = 0;        // tiles issued so far
    unsigned moe_seen = 0;   // POP_MOE_D phases issued in this launch

    // lane 0 only: the stage for the next tile, once the consumers have handed it back.
    // The caller fills it and calls issued().
    __device__ __forceinline__ bool slot(uint8_t*& dst, uint64_t*& full) { return ps_slot(a, s, rp, seq, dst, full); }
    __device__ __forceinline__ void issued() {
        ++seq;
        rp.advance(a.n_stages);
    }
    __device__ __forceinline__ bool one(const uint8_t* src, uint32_t bytes) {
        uint8_t* dst;
        uint64_t* full;
        if (!slot(dst, full)) return false;
        mbar_expect_tx(full, bytes);
        tma_load_1d(dst, src, bytes, full);
        issued();
        return true;
    }

    __device__ bool mamba_a(const PLayer& L, int op_index) {
        if (lane != 0) return true;
        const int64_t rb = row_bytes_of(KIND, a.d);
        const int k = a.dconv, win = k - 1;
        const int nbc = ps_mamba_bc_tiles(a), nconv_tiles = (2 * a.d_state) / 16, ntiles = nbc + a.d_inner / PS_UNIT;
        for (int t = ps_rot(op_index); t < ntiles; t += gridDim.x) {
            uint8_t* dst;
            uint64_t* full;
            if (!slot(dst, full)) return false;
            if (t < nbc) {
                const int r0 = 2 * a.d_inner + t * 16, rows = min(16, a.proj - r0);
                const uint32_t wb = (uint32_t)(rows * rb);
                if (t < nconv_tiles) {
                    const PTileExtra e = ps_bc_extra(a, (int)rb);
                    const int c0 = r0 - a.d_inner;
                    const uint32_t tb = 16u * k * 4u, sb = 16u * win * 4u, bb = L.conv_b ? 64u : 0u;
                    mbar_expect_tx(full, wb + tb + sb + bb);
                    tma_load_1d(dst + e.taps, L.conv_w + (int64_t)c0 * k, tb, full);
                    if (sb) tma_load_1d(dst + e.window, L.conv_state + (int64_t)c0 * win, sb, full);
                    if (bb) tma_load_1d(dst + e.bias, L.conv_b + c0, bb, full);
                } else {
                    mbar_expect_tx(full, wb);
                }
                tma_load_1d(dst, L.mamba_in + r0 * rb, wb, full);
            } else {
                const int u = t - nbc, c0 = u * PS_UNIT;
                const PTileExtra e = ps_unit_extra(a, (int)rb);
                const uint32_t wb = (uint32_t)(PS_UNIT * rb), stb = (uint32_t)(PS_UNIT * a.d_state * 4);
                const uint32_t tb = (uint32_t)PS_UNIT * k * 4u, sb = (uint32_t)PS_UNIT * win * 4u, bb = L.conv_b ? 32u : 0u;
                mbar_expect_tx(full, 2 * wb + stb + tb + sb + bb + 32u);
                tma_load_1d(dst, L.mamba_in + (int64_t)c0 * rb, wb, full);
                tma_load_1d(dst + wb, L.mamba_in + ((int64_t)a.d_inner + c0) * rb, wb, full);
                tma_load_1d(dst + e.state, L.ssm_state + (int64_t)c0 * a.d_state, stb, full);
                tma_load_1d(dst + e.taps, L.conv_w + (int64_t)c0 * k, tb, full);
                if (sb) tma_load_1d(dst + e.window, L.conv_state + (int64_t)c0 * win, sb, full);
                if (bb) tma_load_1d(dst + e.bias, L.conv_b + c0, bb, full);
                tma_load_1d(dst + e.norm, L.mamba_norm + c0, 32u, full);
            }
            issued();
        }
        return true;
    }
    __device__ bool rows16(const uint8_t* w, int N, int K, int op_index) {
        if (lane != 0) return true;
        const int64_t rb = row_bytes_of(KIND, K);
        const int ntiles = (N + 15) / 16;
        for (int t = ps_rot(op_index); t < ntiles; t += gridDim.x) {
            const int r0 = t * 16, rows = min(16, N - r0);
            if (!one(w + r0 * rb, (uint32_t)(rows * rb))) return false;
        }
        return true;
    }
    __device__ bool moe_c(const PLayer& L, int op_index) {
        // the selection bias of the routing that follows (static): into shared memory now
        if (L.router_bias)
            for (int e = lane; e < a.ne; e += 32) s.rbias[e] = L.router_bias[e];
        __syncwarp();
        if (lane != 0) return true;
        const int64_t rb = row_bytes_of(KIND, a.d);
        const int n_router = (a.ne + PS_ROUTER_ROWS - 1) / PS_ROUTER_ROWS;
        const int ntiles = n_router + (L.has_shared ? a.SH / PS_UNIT : 0);
        for (int t = ps_rot(op_index); t < ntiles; t += gridDim.x) {
            if (t < n_router) {
                const int rows = min(PS_ROUTER_ROWS, a.ne - t * PS_ROUTER_ROWS);
                if (!one(reinterpret_cast<const uint8_t*>(L.router + (int64_t)t * PS_ROUTER_ROWS * a.d),
                         (uint32_t)rows * a.d * 4))
                    return false;
            } else {
                const int r0 = (t - n_router) * PS_UNIT;
                uint8_t* dst;
                uint64_t* full;
                if (!slot(dst, full)) return false;
                const uint32_t wb = (uint32_t)(PS_UNIT * rb);
                mbar_expect_tx(full, 2 * wb);
                tma_load_1d(dst, L.sh_gate + r0 * rb, wb, full);
                tma_load_1d(dst + wb, L.sh_up + r0 * rb, wb, full);
                issued();
            }
        }
        return true;
    }
    // The whole warp: the shared expert's down rows are requested at once; then the warp
    // waits for the router's logits (one count per expert on rt_flag, raised during the
    // router phase), turns them into (idx, w) and requests the routed tiles - normally
    // while the consumers are still inside the router phase or its barrier.
    __device__ bool moe_d(const PLayer& L, int layer, int op_index) {
        const int d = a.d;
        const int64_t rb_d = row_bytes_of(KIND, d), rb_sh = L.has_shared ? row_bytes_of(KIND, a.SH) : 0;
        const int n_sd = L.has_shared ? (d + 15) / 16 : 0;
        const int per_slot = a.E / PS_UNIT;
        const int ntiles = n_sd + a.K * per_slot;
        int t = ps_rot(op_index);
        int ok = 1;
        ++moe_seen;
        if (lane == 0) {
            for (; t < n_sd; t += gridDim.x) {
                const int r0 = t * 16, rows = min(16, d - r0);
                if (!one(L.sh_down + r0 * rb_sh, (uint32_t)(rows * rb_sh))) { ok = 0; break; }
            }
            const long long t0 = clock64();
            if (ok && !ps_wait_counter(a, a.rt_flag, moe_seen * (unsigned)a.ne, s.c)) ok = 0;
            if (a.trace && (int)blockIdx.x == a.trace_cta)
                a.trace[(size_t)op_index * PS_TRACE_SLOTS + 6] = (unsigned long long)(clock64() - t0);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (!ok) return false;
        int* r_idx = s.c->r_idx[layer & 1];
        float* r_w = s.c->r_w[layer & 1];
        const long long t1 = clock64();
        ps_route_warp(a.logits, L.router_bias ? s.rbias : nullptr, a.ne, a.K, s.r_p, s.r_sel, r_idx, r_w, lane);
        if (a.trace && lane == 0 && (int)blockIdx.x == a.trace_cta)
            a.trace[(size_t)op_index * PS_TRACE_SLOTS + 7] = (unsigned long long)(clock64() - t1);
        __syncwarp();
        if (lane == 0) {
            __threadfence_block();
            s.c->route_gen = layer + 1;
            for (; t < ntiles; t += gridDim.x) {
                const int i = t - n_sd, k = i / per_slot, r0 = (i % per_slot) * PS_UNIT;
                uint8_t* dst;
                uint64_t* full;
                if (!slot(dst, full)) { ok = 0; break; }
                const int64_t row0 = (int64_t)r_idx[k] * a.E + r0;
                const uint32_t wb = (uint32_t)(PS_UNIT * rb_d);
                mbar_expect_tx(full, 2 * wb);
                tma_load_1d(dst, L.gate + row0 * rb_d, wb, full);
                tma_load_1d(dst + wb, L.up + row0 * rb_d, wb, full);
                issued();
            }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        return ok != 0;
    }
    __device__ bool moe_e(const PLayer& L, int layer, int op_index) {
        if (lane != 0) return true;
        const int64_t rb = row_bytes_of(KIND, a.E);
        const int* r_idx = s.c->r_idx[layer & 1];
        const int ntiles = (a.d + 15) / 16;
        for (int t = ps_rot(op_index); t < ntiles; t += gridDim.x) {
            const int r0 = t * 16, rows = min(16, a.d - r0);
            uint8_t* dst;
            uint64_t* full;
            if (!slot(dst, full)) return false;
            const uint32_t wb = (uint32_t)(rows * rb);
            mbar_expect_tx(full, (uint32_t)a.K * wb);
            for (int k = 0; k < a.K; ++k)
                tma_load_1d(dst + (size_t)k * 16 * rb, L.down + ((int64_t)r_idx[k] * a.d + r0) * rb, wb, full);
            issued();
        }
        return true;
    }
    // never leave with copies of this CTA still in flight
    __device__ void drain() {
        if (lane != 0) return;
        const unsigned n = (unsigned)a.n_stages;
        for (unsigned i = seq > n ? seq - n : 0; i < seq; ++i) {
            bool landed = false;
            for (uint32_t it = 0; it < MBAR_SPIN_LIMIT && !landed; ++it) landed = mbar_try_wait(&s.c->full[i % n], (i / n) & 1u);
            if (!landed) { atomicExch(a.status, 1); break; }
        }
    }
};

template <int KIND>
__global__ void __launch_bounds__(PS_THREADS, 1) persist_step_kernel(PArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    PView s;
    s.stages = smem;
    s.c = reinterpret_cast<PCtl*>(smem + a.off_ctl);
    xact_carve<KIND>(s.xa1, smem + a.off_xa1, a.d, 1, true);
    s.xa2_base = smem + a.off_xa2;
    xact_carve<KIND>(s.xa2, s.xa2_base, a.d_inner, 1, false);
    xact_carve<KIND>(s.xa3, smem + a.off_xa3, a.E, a.K, false);
    s.nw = reinterpret_cast<float*>(smem + a.off_nw);
    s.gs = reinterpret_cast<float*>(smem + a.off_gs);
    s.red = reinterpret_cast<float*>(smem + a.off_red);
    s.r_p = reinterpret_cast<float*>(smem + a.off_route);
    s.r_sel = s.r_p + a.ne;
    s.rbias = s.r_sel + a.ne;
    s.bcd = reinterpret_cast<float*>(smem + a.off_bcd);
    s.hp = s.bcd + 2 * a.d_state + a.n_heads;
    const int n_ops = a.op_end - a.op_begin;
    {
        // the phase list of this launch and the layer table: into shared memory once
        uint64_t* prog = reinterpret_cast<uint64_t*>(smem + a.off_prog);
        const int n_lw = a.n_layers * (int)(sizeof(PLayer) / 8);
        const uint64_t* gops = reinterpret_cast<const uint64_t*>(a.ops + a.op_begin);
        const uint64_t* glay = reinterpret_cast<const uint64_t*>(a.layers);
        uint64_t* slay = prog + ((n_ops + 1) & ~1);
        for (int i = threadIdx.x; i < n_ops; i += PS_THREADS) prog[i] = gops[i];
        for (int i = threadIdx.x; i < n_lw; i += PS_THREADS) slay[i] = glay[i];
        s.ops = reinterpret_cast<const POp*>(prog);
        s.layers = reinterpret_cast<const PLayer*>(slay);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < a.n_stages; ++i) {
            mbar_init(&s.c->full[i], 1);
            mbar_init(&s.c->empty[i], PS_CW);
        }
        mbar_fence_init();
        s.c->abort = 0;
        s.c->snap = 0;
        s.c->route_gen = 0;
    }
    __syncthreads();

    if (warp == PS_CW) {
        PProducer<KIND> p{a, s, lane};
        bool ok = true;
        for (int i = 0; i < n_ops && ok; ++i) {
            const POp op = s.ops[i];
            const int oi = a.op_begin + i;
            if (op.op == POP_EMBED) continue;
            const PLayer& L = s.layers[op.layer];
            switch (op.op) {
                case POP_MAMBA_A: ok = p.mamba_a(L, oi); break;
                case POP_MAMBA_B: ok = p.rows16(L.mamba_out, a.d, a.d_inner, oi); break;
                case POP_MOE_C: ok = p.moe_c(L, oi); break;
                case POP_MOE_D: ok = p.moe_d(L, op.layer, oi); break;
                case POP_MOE_E: ok = p.moe_e(L, op.layer, oi); break;
                default: break;
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (!ok) p.drain();
        return;
    }

    // ---- consumers
    xact_zero_row<KIND, PS_CW>(s.xa1);
    xact_zero_row<KIND, PS_CW>(s.xa3);
    PConsumer<KIND> c{a, s, warp, lane};
    c.prefetch(s.ops[0], 0);
    unsigned nbar = 0;
    bool ok = true;
    for (int i = 0; i < n_ops && ok; ++i) {
        const POp op = s.ops[i];
        const int oi = a.op_begin + i;
        const PLayer& L = s.layers[op.layer];
        ps_stamp(a, oi, 0);
        c.cur_op = oi;
        switch (op.op) {
            case POP_EMBED: ok = c.embed(); break;
            case POP_MAMBA_A: ok = c.mamba_a(L, oi); break;
            case POP_MAMBA_B: ok = c.mamba_b(L, oi); break;
            case POP_MOE_C: ok = c.moe_c(L, oi); break;
            case POP_MOE_D: ok = c.moe_d(L, oi); break;
            case POP_MOE_E: ok = c.moe_e(L, op.layer, oi); break;
            default: break;
        }
        ps_stamp(a, oi, 2);
        if (a.trace && threadIdx.x == 0 && (int)blockIdx.x == a.trace_cta) {
            a.trace[(size_t)oi * PS_TRACE_SLOTS + 4] = (unsigned long long)c.wait_cyc;
            a.trace[(size_t)oi * PS_TRACE_SLOTS + 5] = (unsigned long long)c.rows_cyc;
        }
        c.wait_cyc = c.rows_cyc = 0;
        if (ok && i + 1 < n_ops) ok = c.grid_sync(nbar, s.ops[i + 1]);
        ps_stamp(a, oi, 3);
    }
    if (!ok) s.c->abort = 1;      // the producer sees it at its next wait
    // Last CTA out puts the synchronisation words back to zero for the next launch: a CTA
    // counts itself out only after its last look at them.
    consumer_sync<PS_CW>();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(a.done, 1u) == gridDim.x - 1) {
            *a.bar = 0ULL;
            *a.bc_flag = 0u;
            *a.rt_flag = 0u;
            __threadfence();
            *a.done = 0u;
        }
    }
}

// ===========================================================================
// host side
// ===========================================================================
static inline int round128(size_t v) { return (int)((v + 127) / 128 * 128); }

template <int KIND>
static int plan_kind(PArgs& a) {
    const int d = a.d;
    B200_REQUIRE(d % 256 == 0 && a.d_inner % 256 == 0 && a.E % 256 == 0 && (a.SH == 0 || a.SH % 256 == 0),
                 "persistent step: hidden, Mamba inner, expert and shared widths must be multiples of 256");
    B200_REQUIRE(a.d_head % PS_UNIT == 0 && a.d_state % 32 == 0 && a.d_state <= 32 * PS_NS_MAX,
                 "persistent step: d_head %% 8, d_state %% 32, d_state <= 256 required");
    B200_REQUIRE(a.K >= 1 && a.K <= 16 && a.ne >= a.K && a.ne <= 256, "persistent step: K / ne out of range");
    B200_REQUIRE(a.dconv >= 1 && a.dconv <= 8, "persistent step: d_conv out of range");
    B200_REQUIRE(std::max(std::max(d, a.d_inner), std::max(a.SH, a.K * a.E)) <= 16 * PS_CT,
                 "persistent step: an activation vector is longer than the staging holds (%d floats)", 16 * PS_CT);
    const size_t rb_d = row_bytes_of(KIND, d), rb_di = row_bytes_of(KIND, a.d_inner), rb_e = row_bytes_of(KIND, a.E);
    const size_t rb_sh = a.SH ? row_bytes_of(KIND, a.SH) : 0;
    B200_REQUIRE(rb_d % 16 == 0 && rb_di % 16 == 0 && rb_e % 16 == 0 && rb_sh % 16 == 0 &&
                     (PS_UNIT * rb_d) % 16 == 0,
                 "persistent step: weight rows are not multiples of 16 bytes");
    // in_proj unit: weights, state rows, taps, window, bias, norm weight
    size_t stage = 16 * rb_d + (size_t)PS_UNIT * a.d_state * 4 + (size_t)PS_UNIT * (2 * a.dconv + 1) * 4;
    stage = std::max(stage, 16 * rb_d + (size_t)16 * 2 * a.dconv * 4);   // B/C tile
    stage = std::max(stage, 16 * rb_di);                             // out_proj
    stage = std::max(stage, (size_t)PS_ROUTER_ROWS * d * 4);         // router
    stage = std::max(stage, 16 * rb_sh);                             // shared down
    stage = std::max(stage, (size_t)a.K * 16 * rb_e);                // routed down
    a.stage_bytes = round128(stage);
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off += (bytes + 127) / 128 * 128; return (int)o; };
    a.off_xa1 = take(xact_bytes<KIND>(d, 1, true));
    a.off_xa2 = take(xact_bytes<KIND>(std::max(a.d_inner, std::max(a.SH, 32)), 1, false));
    a.off_xa3 = take(xact_bytes<KIND>(a.E, a.K, false));
    a.off_nw = take((size_t)d * 4);
    a.off_gs = take((size_t)PS_ROUTER_ROWS * (d / 4) * 4);
    a.off_red = take((size_t)2 * PS_CW * 16 * 4);
    a.off_route = take((size_t)3 * a.ne * 4);
    a.off_bcd = take((size_t)(2 * a.d_state + 4 * a.n_heads) * 4);
    a.off_prog = take((size_t)(a.max_ops + 2) * sizeof(POp) + (size_t)a.n_layers * sizeof(PLayer));
    a.off_ctl = take(sizeof(PCtl));
    const size_t other = off;
    int ns = PS_MAX_STAGES;
    while (ns > 0 && (size_t)ns * a.stage_bytes + other > (size_t)PS_SMEM_MAX) --ns;
    if (ns < 3)
        return fail(B200_EUNSUPPORTED,
                    "persistent step: tiles of %d bytes leave fewer than three ring stages beside %zu bytes of staging",
                    a.stage_bytes, other);
    a.n_stages = ns;
    const int ring = ns * a.stage_bytes;
    a.off_xa1 += ring; a.off_xa2 += ring; a.off_xa3 += ring; a.off_nw += ring; a.off_gs += ring; a.off_red += ring;
    a.off_route += ring; a.off_bcd += ring; a.off_prog += ring; a.off_ctl += ring;
    a.smem_bytes = ring + (int)other;
    return B200_OK;
}

int persist_plan(PArgs& a, int kind) {
    switch (kind) {
        case 0: return plan_kind<0>(a);
        case 1: return plan_kind<1>(a);
        case 2: return plan_kind<2>(a);
        case 3: return plan_kind<3>(a);
        case KIND_F16: return plan_kind<KIND_F16>(a);
        default: return fail(B200_EUNSUPPORTED, "persistent step: weight kind %d not supported", kind);
    }
}

template <int KIND>
static int launch_kind(const PArgs& a) {
    auto kern = persist_step_kernel<KIND>;
    static bool configured = false;
    if (!configured) {
        B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PS_SMEM_MAX));
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_sms());
    cfg.blockDim = dim3(PS_THREADS);
    cfg.dynamicSmemBytes = (size_t)a.smem_bytes;
    cfg.stream = stream();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // all CTAs resident, or the launch fails
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
    ++g_kernel_launches;
    return B200_OK;
}

int persist_launch(const PArgs& a, int kind) {
    B200_REQUIRE(a.op_end > a.op_begin && a.smem_bytes > 0 && a.n_stages >= 3, "persistent step: not planned");
    B200_REQUIRE(a.op_end - a.op_begin <= a.max_ops, "persistent step: more phases in a launch than planned for");
    switch (kind) {
        case 0: return launch_kind<0>(a);
        case 1: return launch_kind<1>(a);
        case 2: return launch_kind<2>(a);
        case 3: return launch_kind<3>(a);
        case KIND_F16: return launch_kind<KIND_F16>(a);
        default: return fail(B200_EUNSUPPORTED, "persistent step: weight kind %d not supported", kind);
    }
}

}  // namespace b200
