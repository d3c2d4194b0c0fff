// Fused decode-step kernels, part 1: the streamed single-matrix GEMV (RMSNorm
// prologue; store / residual / Mamba in_proj+conv epilogues) and the Mamba-2 state
// update that also emits the gated-norm statistics.
//
// These fuse across the reference's op boundaries (rmsnorm_forward -> linear ->
// add_inplace in Generator::decode_step_logits, inference/generator.cpp:253-436),
// so they are reached only through the decoder's fused mode; the per-op C ABI keeps
// the reference's granularity.  All kernels are launched with programmatic
// dependent launch: barrier set-up, weight streaming and parameter prefetch run
// before griddepcontrol.wait and overlap the predecessor's tail.
#include "fused_common.cuh"

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

// ===========================================================================
// streamed GEMV: y[M,N] = f(x)[M,K] . W^T, M <= 8
// ===========================================================================
template <int KIND, int MT, int PRO, int EPI>
__global__ void __launch_bounds__(SG_THREADS, 2) stream_gemv_kernel(SgArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    Ring ring;
    ring.stages = smem;
    ring.stage_bytes = a.stage_bytes;
    ring.n_stages = a.n_stages;
    ring.status = a.status;
    XAct xa;
    uint8_t* p = xact_carve<KIND>(xa, smem + (size_t)a.n_stages * a.stage_bytes, a.K, MT, PRO == PRO_RMS);
    float* nw_s = reinterpret_cast<float*>(p);                      // [K] when PRO_RMS
    p += (PRO == PRO_RMS ? (size_t)a.K * 4 : 0);
    float* red = reinterpret_cast<float*>(p);
    p += (size_t)RED_FLOATS * 4;
    ring.full = reinterpret_cast<uint64_t*>(p);
    ring.empty = ring.full + SG_MAX_STAGES;
    double* red_d = reinterpret_cast<double*>(ring.empty + SG_MAX_STAGES);
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
                int tile = first + i * step;
                const uint8_t* wseg = a.w;
                int nseg = a.N;
                if (EPI == EPI_STORE && tile >= a.t1) {       // second / third matrix of the launch
                    const bool third = tile >= a.t2;
                    wseg = third ? a.w3 : a.w2;
                    nseg = third ? a.N3 : a.N2;
                    tile -= third ? a.t2 : a.t1;
                }
                const int rows = min(a.rows_per_tile, nseg - tile * a.rows_per_tile);
                const uint32_t bytes = (uint32_t)(rows * a.row_bytes);
                ring.expect(i, bytes);
                ring.copy(i, 0, wseg + (int64_t)tile * a.rows_per_tile * a.row_bytes, bytes);
                issued = i + 1;
            }
            ring.drain(issued);
        }
        return;
    }

    // consumers: everything independent of the previous kernel first
    if (PRO == PRO_RMS)
        for (int k = threadIdx.x; k < a.K; k += SG_CTHREADS) nw_s[k] = a.norm_w[k];
    xact_zero_row<KIND>(xa);
    pdl_wait();
    // element (row, token) this thread finishes
    const int e_row = threadIdx.x >> 3, e_m = threadIdx.x & 7;
    float in_scale = 1.0f;
    for (int m = 0; m < a.M; ++m) {
        const float* xm = a.x + (int64_t)m * a.x_stride;
        if (a.in_partials) {
            // gated-norm statistic: inv = 1/sqrt(mean + eps) from the scan kernel's block
            // partial sums, reduced together with the activation staging
            double t = 0.0;
            for (int i = threadIdx.x; i < a.n_partials; i += SG_CTHREADS) t += a.in_partials[(int64_t)m * a.n_partials + i];
            t = stage_x<KIND, PRO == PRO_RMS, true>(xm, nw_s, xa, m, a.eps, red_d, t) / (double)a.in_dim;
            if (e_m == m) in_scale = 1.0f / sqrtf((float)t + a.eps);
        } else {
            stage_x<KIND, PRO == PRO_RMS, false>(xm, nw_s, xa, m, a.eps, red_d, 0.0);
        }
    }

    for (int i = 0; i < n_my; ++i) {
        int tile = first + i * step;
        int nseg = a.N;
        float* yseg = a.y;
        int ystride = a.y_stride;
        if (EPI == EPI_STORE && tile >= a.t1) {
            const bool third = tile >= a.t2;
            nseg = third ? a.N3 : a.N2;
            yseg = third ? a.y3 : a.y2;
            ystride = third ? a.y3_stride : a.y2_stride;
            tile -= third ? a.t2 : a.t1;
        }
        const int rows = min(a.rows_per_tile, nseg - tile * a.rows_per_tile);
        const int n = tile * a.rows_per_tile + e_row;
        const bool owner = e_row < rows && e_m < a.M;
        // epilogue operands are fetched before the dot products so their latency hides
        float pre = 0.0f, st[4] = {0, 0, 0, 0}, wc[5] = {0, 0, 0, 0, 0};
        float* dst = nullptr;
        const bool is_conv = EPI == EPI_INPROJ && n >= a.p.d_inner && n < a.p.d_inner + a.p.conv_dim;
        if (owner) {
            if (EPI == EPI_RESIDUAL) {
                dst = a.resid + (int64_t)e_m * a.y_stride + n;
                pre = *dst;
            } else if (is_conv && a.p.k <= 5) {
                const int c = n - a.p.d_inner, win = a.p.k - 1;
                const float* sp = a.conv_state + ((int64_t)e_m * a.p.conv_dim + c) * win;
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
        if (!ring.wait_full(i)) break;
        float* red_pass = red + (size_t)(i & 1) * RED_BUF;
        tile_compute<KIND, MT>(ring.stage(i), a.row_bytes, rows, a.K, xa, 0, a.M, red_pass, warp, lane);
        ring.release(i);
        consumer_sync();
        if (owner) {
            float v = red_value<KIND>(red_pass, e_row, e_m) * in_scale;
            const int m = e_m;
            if (EPI == EPI_STORE) {
                yseg[(int64_t)m * ystride + n] = v * a.out_scale;
            } else if (EPI == EPI_RESIDUAL) {
                *dst = pre + v * a.res_mult;
            } else {
                // Mamba in_proj row n: gate | conv channel (window of raw inputs, oldest
                // first; unfused ops in the reference's order) | dt
                const MambaDims& p = a.p;
                if (n < p.d_inner) {
                    a.gate[(int64_t)m * p.d_inner + n] = v;
                } else if (is_conv) {
                    const int c = n - p.d_inner, win = p.k - 1;
                    float* sp = a.conv_state + ((int64_t)m * p.conv_dim + c) * win;
                    float t;
                    if (p.k <= 5) {
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
}

// ===========================================================================
// Mamba-2 state update (decode) + gated-norm statistics
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
// host side
// ===========================================================================
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

template <int KIND, int PRO, int EPI>
static int launch_sg_mt(SgArgs a, int grid) {
    const int mt = a.M == 1 ? 1 : a.M == 2 ? 2 : a.M <= 4 ? 4 : 8;
    const size_t other = xact_bytes<KIND>(a.K, mt, PRO == PRO_RMS) + (PRO == PRO_RMS ? (size_t)a.K * 4 : 0) +
                         (size_t)RED_FLOATS * 4 + BAR_BYTES;
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
    const int R = pick_rows(kind, a.row_bytes, a.row_bytes, a.row_bytes, a.N);
    if (R < 1) return fail(B200_EUNSUPPORTED, "stream_gemv: row size %lld cannot be tiled to 16 bytes", (long long)a.row_bytes);
    if ((R * a.row_bytes) % 16 != 0 || !tail_tile_ok(a.N, R, a.row_bytes))
        return fail(B200_EUNSUPPORTED, "stream_gemv: %d rows of %lld bytes cannot be tiled to 16 bytes", a.N, (long long)a.row_bytes);
    a.rows_per_tile = R;
    a.num_tiles = ceil_div(a.N, R);
    a.t1 = a.t2 = a.num_tiles;
    if (a.N2 > 0 || a.N3 > 0) {
        B200_REQUIRE(epi == EPI_STORE && a.N2 > 0 && a.w2 && a.y2 && (a.N3 == 0 || (a.w3 && a.y3)),
                     "stream_gemv: extra matrices need the store epilogue and their pointers");
        B200_REQUIRE(((reinterpret_cast<uintptr_t>(a.w2) | reinterpret_cast<uintptr_t>(a.w3)) & 15) == 0,
                     "stream_gemv: weights must be 16-byte aligned");
        if (!tail_tile_ok(a.N2, R, a.row_bytes) || (a.N3 > 0 && !tail_tile_ok(a.N3, R, a.row_bytes)))
            return fail(B200_EUNSUPPORTED, "stream_gemv: rows of %lld bytes cannot be tiled to 16 bytes", (long long)a.row_bytes);
        a.t2 = a.t1 + ceil_div(a.N2, R);
        a.num_tiles = a.t2 + ceil_div(a.N3, R);
    }
    a.stage_bytes = (int)((R * a.row_bytes + 127) / 128 * 128);
    a.status = stream_status_ptr();
    B200_REQUIRE(a.status, "stream_gemv: status word allocation failed");
    B200_REQUIRE((reinterpret_cast<uintptr_t>(a.w) & 15) == 0, "stream_gemv: weights must be 16-byte aligned");
    const int grid = std::min(a.num_tiles, num_sms());
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

}  // namespace b200

extern "C" int b200_stream_status(void) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return b200::cuda_status(e, "stream_status: synchronize");
    return b200::stream_status_check("stream_status");
}
