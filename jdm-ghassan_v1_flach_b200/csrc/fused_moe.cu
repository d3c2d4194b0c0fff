// Fused decode-step kernels, part 2: the MoE layer for a few tokens in three
// streamed kernels -
//   phase 1  router logits in the reference's exact fp32 order + the shared
//            expert's gate/up (SwiGLU activation); the CTA that finishes the last
//            router tile does softmax / top-K / mixture weights
//   phase 2  the routed experts' gate/up
//   phase 3  all down projections, weighted combine, residual add
// Arithmetic followed: cpu::moe_forward_bias, core/moe_cpu.cpp:198-288.
#include "fused_common.cuh"
#include "route.cuh"

namespace b200 {

constexpr int ROUTER_ROWS = 4;                // experts per router tile, one per consumer warp (the rest idle)

// Router logit of one expert for one token, exactly as core/moe_cpu.cpp:76-83:
// group sums ((a0b0 + a1b1) + a2b2) + a3b3 by all lanes, then lane 0 adds them in
// order.  wrow: the expert's fp32 router row (shared memory); gs: d/4 floats of
// per-warp scratch.  Valid in lane 0.
template <int KIND>
__device__ __forceinline__ float router_logit(const float* wrow, const XAct& xa, int m, float* gs, int d, int lane) {
    const int groups = d >> 2;
    const float* xf = UsesMma<KIND>::value ? xa.f32 + (size_t)m * d : xa.xs + (size_t)m * xa.xs_tok;
    for (int g = lane; g < groups; g += 32) {
        const float4 b = *reinterpret_cast<const float4*>(wrow + 4 * g);
        const int xi = UsesMma<KIND>::value ? 4 * g : xs_index<KIND>(4 * g);
        const float4 a = *reinterpret_cast<const float4*>(xf + xi);
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
        for (int k = groups << 2; k < d; ++k) {
            const int xi = UsesMma<KIND>::value ? k : xs_index<KIND>(k);
            chain = __fadd_rn(chain, __fmul_rn(xf[xi], wrow[k]));
        }
    }
    __syncwarp();
    return chain;
}

// ---- phase 1 -------------------------------------------------------------------
// tiles [0, n_router): ROUTER_ROWS fp32 router rows; then shared tiles: R rows of
// sh_gate (pass 0) followed by the same R rows of sh_up (pass 1).
template <int KIND, int MT>
__global__ void __launch_bounds__(SG_THREADS, 2) moe_phase1_kernel(MoeFusedArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    Ring ring;
    ring.stages = smem;
    ring.stage_bytes = a.stage_bytes;
    ring.n_stages = a.n_stages;
    ring.status = a.status;
    XAct xa;
    uint8_t* p = xact_carve<KIND>(xa, smem + (size_t)a.n_stages * a.stage_bytes, a.d, MT, true);
    float* nw_s = reinterpret_cast<float*>(p);
    p += (size_t)a.d * 4;
    float* gs = reinterpret_cast<float*>(p);                        // [SG_CONSUMERS][d/4]
    p += (size_t)SG_CONSUMERS * (a.d >> 2) * 4;
    float* r_p = reinterpret_cast<float*>(p);           // routing scratch: [ne] [ne] [16] [16]
    float* r_sel = r_p + a.ne;
    float* r_w = r_sel + a.ne;
    int* r_idx = reinterpret_cast<int*>(r_w + 16);
    p = reinterpret_cast<uint8_t*>(r_idx + 16);
    p = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 15) & ~(uintptr_t)15);
    float* red = reinterpret_cast<float*>(p);
    p += (size_t)RED_FLOATS * 4;
    ring.full = reinterpret_cast<uint64_t*>(p);
    ring.empty = ring.full + SG_MAX_STAGES;
    double* red_d = reinterpret_cast<double*>(ring.empty + SG_MAX_STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_router = (a.ne + ROUTER_ROWS - 1) / ROUTER_ROWS;
    const int n_shared = a.SH > 0 ? (a.SH + a.rows_per_tile - 1) / a.rows_per_tile : 0;
    const int num_tiles = n_router + n_shared;
    const int first = blockIdx.x, step = gridDim.x;
    const int n_my = first < num_tiles ? (num_tiles - first + step - 1) / step : 0;
    const int64_t rb = row_bytes_of(KIND, a.d);
    const int sub = a.rows_per_tile * (int)rb;
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
                    ring.copy(i, sub, a.sh_u + r0 * rb, bytes);
                }
                issued = i + 1;
            }
            ring.drain(issued);
        }
        return;
    }
    for (int k = threadIdx.x; k < a.d; k += SG_CTHREADS) nw_s[k] = a.norm_w[k];
    xact_zero_row<KIND>(xa);
    pdl_wait();
    for (int m = 0; m < a.M; ++m) stage_x<KIND, true, false>(a.x + (int64_t)m * a.d, nw_s, xa, m, a.eps, red_d, 0.0);
    const int e_row = threadIdx.x >> 3, e_m = threadIdx.x & 7;

    for (int i = 0; i < n_my; ++i) {
        if (!ring.wait_full(i)) break;
        const int tile = first + i * step;
        const uint8_t* ts = ring.stage(i);
        if (tile < n_router) {
            const int e = tile * ROUTER_ROWS + warp;
            if (warp < ROUTER_ROWS && e < a.ne) {
                const float* wrow = reinterpret_cast<const float*>(ts) + (int64_t)warp * a.d;
                for (int m = 0; m < a.M; ++m) {
                    const float lg = router_logit<KIND>(wrow, xa, m, gs + warp * (a.d >> 2), a.d, lane);
                    if (lane == 0) a.logits[(int64_t)m * a.ne + e] = lg;
                }
                if (lane == 0) __threadfence();
            }
            ring.release(i);
            consumer_sync();       // keeps the tile parity of the reduction buffers in step
            // The CTA that completes the last router tile turns the logits into (idx, w):
            // nobody waits - each tile counts itself in, and whoever counts last finds every
            // logit published (fence before the count, fence after it).
            if (warp == 0) {
                int last = 0;
                if (lane == 0) {
                    __threadfence();
                    last = atomicAdd(a.route_counter, 1) == n_router - 1;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence();
                    for (int m = 0; m < a.M; ++m) {
                        route_finish_warp(a.logits + (int64_t)m * a.ne, a.router_bias, a.ne, a.K, r_p, r_sel, r_idx, r_w,
                                          a.probs_out ? a.probs_out + (int64_t)m * a.ne : nullptr, lane);
                        if (lane < a.K) {
                            a.idx[(int64_t)m * a.K + lane] = r_idx[lane];
                            a.w[(int64_t)m * a.K + lane] = r_w[lane];
                        }
                        __syncwarp();
                    }
                    if (lane == 0) *a.route_counter = 0;       // ready for the next layer
                }
            }
        } else {
            const int r0 = (tile - n_router) * a.rows_per_tile;
            const int rows = min(a.rows_per_tile, a.SH - r0);
            float* red_buf = red + (size_t)(i & 1) * RED_BUF;
            tile_compute<KIND, MT>(ts, rb, rows, a.d, xa, 0, a.M, red_buf, warp, lane);
            tile_compute<KIND, MT>(ts + sub, rb, rows, a.d, xa, 0, a.M, red_buf + RED_PASS, warp, lane);
            ring.release(i);
            consumer_sync();
            if (e_row < rows && e_m < a.M) {
                const float g = red_value<KIND>(red_buf, e_row, e_m);
                const float u = red_value<KIND>(red_buf + RED_PASS, e_row, e_m);
                a.sh_act[(int64_t)e_m * a.SH + r0 + e_row] = silu_acc(g) * u;
            }
        }
    }
}

// ---- phase 2 -------------------------------------------------------------------
// grid (ctas, M): blockIdx.y is the token.  The producer warp reads the experts
// phase 1 chose and streams tiles (k, row tile) of expert idx[k]: R gate rows then R
// up rows.
template <int KIND>
__global__ void __launch_bounds__(SG_THREADS, 2) moe_phase2_kernel(MoeFusedArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    Ring ring;
    ring.stages = smem;
    ring.stage_bytes = a.stage_bytes;
    ring.n_stages = a.n_stages;
    ring.status = a.status;
    XAct xa;
    uint8_t* p = xact_carve<KIND>(xa, smem + (size_t)a.n_stages * a.stage_bytes, a.d, 1, true);
    float* nw_s = reinterpret_cast<float*>(p);
    p += (size_t)a.d * 4;
    int* s_idx = reinterpret_cast<int*>(p);             // [16]
    p = reinterpret_cast<uint8_t*>(s_idx + 16);
    p = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 15) & ~(uintptr_t)15);
    float* red = reinterpret_cast<float*>(p);
    p += (size_t)RED_FLOATS * 4;
    ring.full = reinterpret_cast<uint64_t*>(p);
    ring.empty = ring.full + SG_MAX_STAGES;
    double* red_d = reinterpret_cast<double*>(ring.empty + SG_MAX_STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.y;
    const int tiles_per_slot = (a.E + a.rows_per_tile - 1) / a.rows_per_tile;
    const int num_tiles = a.K * tiles_per_slot;
    const int first = blockIdx.x, step = gridDim.x;
    const int n_my = first < num_tiles ? (num_tiles - first + step - 1) / step : 0;
    const int64_t rb = row_bytes_of(KIND, a.d);
    const int sub = a.rows_per_tile * (int)rb;
    ring.init();
    if (threadIdx.x == 0) pdl_launch_dependents();

    if (warp == SG_CONSUMERS) {
        pdl_wait();
        if (lane < a.K) s_idx[lane] = a.idx[(int64_t)m * a.K + lane];     // chosen by phase 1
        __syncwarp();
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
                ring.copy(i, sub, a.ups + row0 * rb, bytes);
                issued = i + 1;
            }
            ring.drain(issued);
        }
        return;
    }
    for (int k = threadIdx.x; k < a.d; k += SG_CTHREADS) nw_s[k] = a.norm_w[k];
    xact_zero_row<KIND>(xa);
    pdl_wait();
    stage_x<KIND, true, false>(a.x + (int64_t)m * a.d, nw_s, xa, 0, a.eps, red_d, 0.0);
    const int e_row = threadIdx.x >> 3, e_m = threadIdx.x & 7;
    for (int i = 0; i < n_my; ++i) {
        if (!ring.wait_full(i)) break;
        const int tile = first + i * step;
        const int k = tile / tiles_per_slot, r0 = (tile % tiles_per_slot) * a.rows_per_tile;
        const int rows = min(a.rows_per_tile, a.E - r0);
        const uint8_t* ts = ring.stage(i);
        float* red_buf = red + (size_t)(i & 1) * RED_BUF;
        tile_compute<KIND, 1>(ts, rb, rows, a.d, xa, 0, 1, red_buf, warp, lane);
        tile_compute<KIND, 1>(ts + sub, rb, rows, a.d, xa, 0, 1, red_buf + RED_PASS, warp, lane);
        ring.release(i);
        consumer_sync();
        if (e_row < rows && e_m == 0) {
            const float g = red_value<KIND>(red_buf, e_row, 0);
            const float u = red_value<KIND>(red_buf + RED_PASS, e_row, 0);
            a.act[((int64_t)m * a.K + k) * a.E + r0 + e_row] = silu_acc(g) * u;
        }
    }
}

// ---- phase 3 -------------------------------------------------------------------
// grid (ctas, M).  A tile is R output rows: R rows of sh_down (K = SH) followed, for
// each k, by R rows of down[idx[k]] (K = E).  The routed activations are staged as K
// "tokens" of one activation block so every slot has its own vector.
template <int KIND>
__global__ void __launch_bounds__(SG_THREADS, 2) moe_phase3_kernel(MoeFusedArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    Ring ring;
    ring.stages = smem;
    ring.stage_bytes = a.stage_bytes;
    ring.n_stages = a.n_stages;
    ring.status = a.status;
    XAct xsh, xe;
    uint8_t* p = smem + (size_t)a.n_stages * a.stage_bytes;
    if (a.SH > 0) p = xact_carve<KIND>(xsh, p, a.SH, 1, false);
    p = xact_carve<KIND>(xe, p, a.E, a.K, false);
    float* s_w = reinterpret_cast<float*>(p);       // [16]
    p += 64;
    float* red = reinterpret_cast<float*>(p);
    p += (size_t)RED_FLOATS * 4;
    ring.full = reinterpret_cast<uint64_t*>(p);
    ring.empty = ring.full + SG_MAX_STAGES;
    double* red_d = reinterpret_cast<double*>(ring.empty + SG_MAX_STAGES);
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
    if (a.SH > 0) xact_zero_row<KIND>(xsh);
    xact_zero_row<KIND>(xe);
    pdl_wait();
    if (threadIdx.x < a.K) s_w[threadIdx.x] = a.w[(int64_t)m * a.K + threadIdx.x];
    if (a.SH > 0) stage_x<KIND, false, false>(a.sh_act + (int64_t)m * a.SH, nullptr, xsh, 0, 0.0f, red_d, 0.0);
    stage_rows<KIND>(a.act + (int64_t)m * a.K * a.E, a.E, xe, a.K, red_d);
    const int e_row = threadIdx.x >> 3, e_m = threadIdx.x & 7;
    for (int i = 0; i < n_my; ++i) {
        const int r0 = (first + i * step) * a.rows_per_tile;
        const int rows = min(a.rows_per_tile, a.d - r0);
        const bool owner = e_row < rows && e_m == 0;
        float* dst = a.resid + (int64_t)m * a.d + r0 + e_row;
        float pre = 0.0f;
        if (owner) pre = *dst;
        if (!ring.wait_full(i)) break;
        const uint8_t* ts = ring.stage(i);
        float* red_buf = red + (size_t)(i & 1) * RED_BUF;
        if (UsesMma<KIND>::value) {
            // combine in registers: fragment-wise sum of shared + w_k * routed_k
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            if (a.SH > 0) {
                const XHalf xh = xsh.half();
                if (KIND == 3) tile_dot_q4k(ts, (int)rb_sh, a.SH, xh, 1, warp, SG_CONSUMERS, lane, acc);
                else tile_dot_f16(ts, (int)rb_sh, a.SH, xh, 1, warp, SG_CONSUMERS, lane, acc);
            }
            for (int k = 0; k < a.K; ++k) {
                XHalf xh = xe.half();
                xh.hi += (size_t)k * xh.stride;
                xh.lo += (size_t)k * xh.stride;
                xh.sumx += (size_t)k * xh.nsub;
                xh.zero_row -= k;
                float t[4] = {0.f, 0.f, 0.f, 0.f};
                if (KIND == 3) tile_dot_q4k(ts + sub_sh + k * sub_e, (int)rb_e, a.E, xh, 1, warp, SG_CONSUMERS, lane, t);
                else tile_dot_f16(ts + sub_sh + k * sub_e, (int)rb_e, a.E, xh, 1, warp, SG_CONSUMERS, lane, t);
                const float wk = s_w[k];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] += wk * t[j];
            }
            float* o = red_buf + (size_t)warp * RED_PASSES * RED_PASS;
            const int gid = lane >> 2, c = 2 * (lane & 3);
            o[gid * RED_TOK + c] = acc[0];
            o[gid * RED_TOK + c + 1] = acc[1];
            o[(gid + 8) * RED_TOK + c] = acc[2];
            o[(gid + 8) * RED_TOK + c + 1] = acc[3];
        } else {
            for (int r = warp; r < rows; r += SG_CONSUMERS) {
                float acc = 0.0f, t[1];
                if (a.SH > 0) {
                    row_dot_xs<KIND, 1>(ts + (int64_t)r * rb_sh, xsh.xs, xsh.xs_tok, 1, a.SH, lane, t);
                    acc = t[0];
                }
                for (int k = 0; k < a.K; ++k) {
                    row_dot_xs<KIND, 1>(ts + sub_sh + k * sub_e + (int64_t)r * rb_e, xe.xs + (size_t)k * xe.xs_tok,
                                        xe.xs_tok, 1, a.E, lane, t);
                    acc = __fadd_rn(acc, __fmul_rn(s_w[k], t[0]));
                }
                if (lane == 0) red_buf[r * RED_TOK] = acc;
            }
        }
        ring.release(i);
        consumer_sync();
        if (owner) *dst = pre + red_value<KIND>(red_buf, e_row, 0) * a.res_mult;
    }
}

// ===========================================================================
// host side
// ===========================================================================
template <int KIND>
static int moe_fused_kind(MoeFusedArgs a) {
    const int64_t rb_d = row_bytes_of(KIND, a.d), rb_e = row_bytes_of(KIND, a.E);
    const int64_t rb_sh = a.SH > 0 ? row_bytes_of(KIND, a.SH) : 0;
    const int mt = a.M == 1 ? 1 : a.M == 2 ? 2 : a.M <= 4 ? 4 : 8;
    const size_t fixed = (size_t)RED_FLOATS * 4 + BAR_BYTES + 64;
    int rc;
    // ---- phase 1
    {
        MoeFusedArgs p1 = a;
        const int R = pick_rows(KIND, 2 * rb_d, rb_d, rb_d, std::max(a.SH, 1));
        if (R < 1 || !tail_tile_ok(a.SH, R, rb_d)) return fail(B200_EUNSUPPORTED, "moe_fused: row size cannot be tiled to 16 bytes");
        p1.rows_per_tile = R;
        const size_t stage = std::max<size_t>((size_t)ROUTER_ROWS * a.d * 4, (size_t)2 * R * rb_d);
        p1.stage_bytes = (int)((stage + 127) / 128 * 128);
        const size_t other = xact_bytes<KIND>(a.d, mt, true) + (size_t)a.d * 4 + (size_t)SG_CONSUMERS * (a.d / 4) * 4 +
                             (size_t)2 * a.ne * 4 + 128 + 16 + fixed;
        p1.n_stages = pick_stages(p1.stage_bytes, other);
        if (p1.n_stages < 2) return fail(B200_EUNSUPPORTED, "moe_fused: hidden size %d does not fit the shared-memory staging", a.d);
        const int tiles = ceil_div(a.ne, ROUTER_ROWS) + (a.SH > 0 ? ceil_div(a.SH, R) : 0);
        const size_t smem = (size_t)p1.n_stages * p1.stage_bytes + other;
        const int grid = std::min(tiles, num_sms());
#define P1(MT_)                                                                 \
    {                                                                           \
        auto kern = moe_phase1_kernel<KIND, MT_>;                               \
        static bool cfgd = false;                                               \
        rc = B200_OK;                                                           \
        if (!cfgd) { rc = allow_smem(kern); cfgd = (rc == B200_OK); }           \
        if (!rc) rc = launch_pdl(kern, dim3(grid), dim3(SG_THREADS), smem, p1); \
    }
        if (mt == 1) P1(1) else if (mt == 2) P1(2) else if (mt == 4) P1(4) else P1(8)
#undef P1
        if (rc) return rc;
    }
    // ---- phase 2
    {
        MoeFusedArgs p2 = a;
        const int R = pick_rows(KIND, 2 * rb_d, rb_d, rb_d, a.E);
        if (R < 1 || !tail_tile_ok(a.E, R, rb_d)) return fail(B200_EUNSUPPORTED, "moe_fused: row size cannot be tiled to 16 bytes");
        p2.rows_per_tile = R;
        p2.stage_bytes = (int)(((size_t)2 * R * rb_d + 127) / 128 * 128);
        const size_t other = xact_bytes<KIND>(a.d, 1, true) + (size_t)a.d * 4 + 64 + 16 + fixed;
        p2.n_stages = pick_stages(p2.stage_bytes, other);
        if (p2.n_stages < 2) return fail(B200_EUNSUPPORTED, "moe_fused: hidden size %d does not fit the shared-memory staging", a.d);
        const int tiles = a.K * ceil_div(a.E, R);
        const int grid = std::max(1, std::min(tiles, num_sms() / std::max(1, a.M)));
        auto kern = moe_phase2_kernel<KIND>;
        static bool cfgd = false;
        if (!cfgd) { rc = allow_smem(kern); if (rc) return rc; cfgd = true; }
        rc = launch_pdl(kern, dim3(grid, a.M), dim3(SG_THREADS), (size_t)p2.n_stages * p2.stage_bytes + other, p2);
        if (rc) return rc;
    }
    // ---- phase 3
    {
        MoeFusedArgs p3 = a;
        const int64_t per_row = rb_sh + (int64_t)a.K * rb_e;
        const int R = pick_rows(KIND, per_row, rb_e, rb_sh > 0 ? rb_sh : rb_e, a.d);
        if (R < 1 || (R * rb_e) % 16 != 0 || (R * rb_sh) % 16 != 0 || !tail_tile_ok(a.d, R, rb_e, rb_sh))
            return fail(B200_EUNSUPPORTED, "moe_fused: row size cannot be tiled to 16 bytes");
        p3.rows_per_tile = R;
        p3.stage_bytes = (int)(((size_t)R * per_row + 127) / 128 * 128);
        const size_t other = (a.SH > 0 ? xact_bytes<KIND>(a.SH, 1, false) : 0) + xact_bytes<KIND>(a.E, a.K, false) + fixed;
        p3.n_stages = pick_stages(p3.stage_bytes, other);
        if (p3.n_stages < 2) return fail(B200_EUNSUPPORTED, "moe_fused: expert width does not fit the shared-memory staging");
        const int tiles = ceil_div(a.d, R);
        const int grid = std::max(1, std::min(tiles, num_sms() / std::max(1, a.M)));
        auto kern = moe_phase3_kernel<KIND>;
        static bool cfgd = false;
        if (!cfgd) { rc = allow_smem(kern); if (rc) return rc; cfgd = true; }
        rc = launch_pdl(kern, dim3(grid, a.M), dim3(SG_THREADS), (size_t)p3.n_stages * p3.stage_bytes + other, p3);
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
    a.route_counter = a.status ? a.status + 8 : nullptr;      // a word of the same zero-initialised block
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
