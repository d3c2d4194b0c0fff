// Fused decode-step kernels (batch <= 8 tokens): weight-streaming GEMV with the
// preceding RMSNorm as prologue and the conv step / residual add as epilogue, and
// the Mamba-2 state update that also produces the gated-norm statistics.
//
// These fuse across the reference's op boundaries (rmsnorm_forward -> linear ->
// add_inplace in Generator::decode_step_logits, inference/generator.cpp:253-436),
// so they are reached only through the decoder's fused mode; the per-op C ABI keeps
// the reference's granularity.
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
constexpr int SG_THREADS = (SG_CONSUMERS + 1) * 32;
constexpr int SG_STAGES = 4;

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(SG_CONSUMERS * 32) : "memory"); }

// Sum over the consumer warps (threads 0..127); result in every consumer thread.
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

template <int KIND, int MT, int PRO, int EPI>
__global__ void __launch_bounds__(SG_THREADS) stream_gemv_kernel(SgArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stages = smem;
    float* xs = reinterpret_cast<float*>(smem + (size_t)SG_STAGES * a.stage_bytes);
    const int xs_tok = xs_floats(a.K);
    uint64_t* full = reinterpret_cast<uint64_t*>(xs + (size_t)MT * xs_tok);
    uint64_t* empty = full + SG_STAGES;
    double* red = reinterpret_cast<double*>(empty + SG_STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first = blockIdx.x, step = gridDim.x;
    const int n_my = first < a.num_tiles ? (a.num_tiles - first + step - 1) / step : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SG_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], SG_CONSUMERS);
        }
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) pdl_launch_dependents();

    if (warp == SG_CONSUMERS) {
        // ---- producer: weights do not depend on the previous kernel, start at once
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < n_my; ++i) {
                const int s = i % SG_STAGES;
                if (i >= SG_STAGES && !mbar_wait(&empty[s], ((i / SG_STAGES) - 1) & 1, a.status)) break;
                const int tile = first + i * step;
                const int rows = min(a.rows_per_tile, a.N - tile * a.rows_per_tile);
                const uint32_t bytes = (uint32_t)(rows * a.row_bytes);
                mbar_expect_tx(&full[s], bytes);
                tma_load_1d(stages + (size_t)s * a.stage_bytes, a.w + (int64_t)tile * a.rows_per_tile * a.row_bytes,
                            bytes, &full[s]);
                issued = i + 1;
            }
            // never leave with copies of this CTA still in flight
            for (int i = max(0, issued - SG_STAGES); i < issued; ++i)
                if (!mbar_wait(&full[i % SG_STAGES], (i / SG_STAGES) & 1, a.status)) break;
        }
        return;
    }

    // ---- consumers: wait for the previous kernel, stage the activations
    pdl_wait();
    for (int m = 0; m < a.M; ++m) {
        const float* xm = a.x + (int64_t)m * a.x_stride;
        float inv = 1.0f;
        if (PRO == PRO_RMS) {
            double ss = 0.0;
            for (int k = threadIdx.x; k < a.K; k += SG_CONSUMERS * 32) {
                const double v = (double)xm[k];
                ss += v * v;
            }
            ss = consumer_sum_d(ss, red);
            const double inv_d = 1.0 / sqrt(ss / (double)a.K + (double)a.eps);
            inv = isfinite(inv_d) ? (float)inv_d : 0.0f;
        }
        for (int k = threadIdx.x; k < a.K; k += SG_CONSUMERS * 32) {
            float v = xm[k];
            if (PRO == PRO_RMS) v = v * inv * a.norm_w[k];
            xs[m * xs_tok + xs_index<KIND>(k)] = v;
        }
    }
    consumer_sync();

    for (int i = 0; i < n_my; ++i) {
        const int s = i % SG_STAGES;
        if (!mbar_wait(&full[s], (i / SG_STAGES) & 1, a.status)) break;
        const int tile = first + i * step;
        const int rows = min(a.rows_per_tile, a.N - tile * a.rows_per_tile);
        const uint8_t* tile_smem = stages + (size_t)s * a.stage_bytes;
        for (int r = warp; r < rows; r += SG_CONSUMERS) {
            float acc[MT];
            row_dot_xs<KIND, MT>(tile_smem + (int64_t)r * a.row_bytes, xs, xs_tok, a.M, a.K, lane, acc);
            const int n = tile * a.rows_per_tile + r;
            if (lane < MT && lane < a.M) {
                float v = 0.0f;
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m == lane) v = acc[m];
                const int m = lane;
                if (a.in_scale) v *= a.in_scale[m];
                if (EPI == EPI_STORE) {
                    a.y[(int64_t)m * a.y_stride + n] = v * a.out_scale;
                } else if (EPI == EPI_RESIDUAL) {
                    float* dst = a.resid + (int64_t)m * a.y_stride + n;
                    *dst = *dst + v * a.res_mult;
                } else {
                    // in_proj row n: gate | conv channel | dt  (see mamba_inproj_conv_kernel)
                    const MambaDims& p = a.p;
                    if (n < p.d_inner) {
                        a.gate[(int64_t)m * p.d_inner + n] = v;
                    } else if (n < p.d_inner + p.conv_dim) {
                        const int c = n - p.d_inner, win = p.k - 1;
                        float* st = a.conv_state + ((int64_t)m * p.conv_dim + c) * win;
                        const float* wc = a.conv_w + (int64_t)c * p.k;
                        float t = a.conv_b ? a.conv_b[c] : 0.0f;
                        for (int j = 0; j < win; ++j) {
                            const float sv = st[j];
                            t = __fadd_rn(t, __fmul_rn(wc[j], sv));
                            if (j > 0) st[j - 1] = sv;
                        }
                        t = __fadd_rn(t, __fmul_rn(wc[win], v));
                        if (win > 0) st[win - 1] = v;
                        a.bc[(int64_t)m * p.conv_dim + c] = silu_acc(t);
                    } else {
                        a.dt_raw[(int64_t)m * p.n_heads + (n - p.d_inner - p.conv_dim)] = v;
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
}

// ---------------------------------------------------------------------------
// Mamba-2 state update (decode) that also prepares the gated norm: writes
// u = y * silu(gate) * norm_w and, through a last-block-done counter, the scalar
// inv = 1/sqrt(mean((y*silu(gate))^2) + eps) per sequence; the out-projection then
// computes inv * (W u).  The block partial sums are added in block order, so the
// result does not depend on scheduling.
// ---------------------------------------------------------------------------
constexpr int FS_WARPS = 8;
__global__ void __launch_bounds__(FS_WARPS * 32)
mamba_scan_norm_kernel(const float* __restrict__ bc, const float* __restrict__ dt_raw,
                       const float* __restrict__ gate, const float* __restrict__ dt_bias,
                       const float* __restrict__ a_log, const float* __restrict__ Dv,
                       const float* __restrict__ norm_w, float* __restrict__ ssm_state,
                       float* __restrict__ u_out, double* __restrict__ partials, unsigned* __restrict__ counter,
                       float* __restrict__ inv_out, MambaDims p) {
    __shared__ double wsum[FS_WARPS];
    __shared__ bool last;
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows = p.n_heads * p.d_head;
    const int row = blockIdx.x * FS_WARPS + warp;
    const int m = blockIdx.y;
    double sq = 0.0;
    if (row < rows) {
        const int h = row / p.d_head;
        const float uu = dt_raw[(int64_t)m * p.n_heads + h] + dt_bias[h];
        const float dt = (uu > 20.0f) ? uu : log1pf(expf(uu));
        const float A = -expf(a_log[h]);
        const float dA = expf(__fmul_rn(A, dt));
        const float* bcm = bc + (int64_t)m * p.conv_dim;
        const float xv = bcm[row];
        const float* Bv = bcm + p.d_inner;
        const float* Cv = Bv + p.d_state;
        float* s = ssm_state + ((int64_t)m * rows + row) * p.d_state;
        float acc = 0.0f;
        if ((p.d_state & 127) == 0) {
            for (int j = lane * 4; j < p.d_state; j += 128) {
                float4 sv = *reinterpret_cast<float4*>(s + j);
                const float4 b = *reinterpret_cast<const float4*>(Bv + j);
                const float4 c = *reinterpret_cast<const float4*>(Cv + j);
                sv.x = __fadd_rn(__fmul_rn(dA, sv.x), __fmul_rn(__fmul_rn(dt, b.x), xv));
                sv.y = __fadd_rn(__fmul_rn(dA, sv.y), __fmul_rn(__fmul_rn(dt, b.y), xv));
                sv.z = __fadd_rn(__fmul_rn(dA, sv.z), __fmul_rn(__fmul_rn(dt, b.z), xv));
                sv.w = __fadd_rn(__fmul_rn(dA, sv.w), __fmul_rn(__fmul_rn(dt, b.w), xv));
                *reinterpret_cast<float4*>(s + j) = sv;
                acc += c.x * sv.x + c.y * sv.y + c.z * sv.z + c.w * sv.w;
            }
        } else {
            for (int j = lane; j < p.d_state; j += 32) {
                const float sn = __fadd_rn(__fmul_rn(dA, s[j]), __fmul_rn(__fmul_rn(dt, Bv[j]), xv));
                s[j] = sn;
                acc += Cv[j] * sn;
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            const float y = acc + Dv[h] * xv;
            const float g = gate[(int64_t)m * p.d_inner + row];
            const float v = y * silu_acc(g);
            u_out[(int64_t)m * p.d_inner + row] = v * norm_w[row];
            sq = (double)v * v;
        }
    }
    if (lane == 0) wsum[warp] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < FS_WARPS; ++w) t += wsum[w];
        partials[(int64_t)m * gridDim.x + blockIdx.x] = t;
        __threadfence();
        const unsigned done = atomicAdd(&counter[m], 1u);
        last = (done == gridDim.x - 1);
    }
    __syncthreads();
    if (last && threadIdx.x == 0) {
        __threadfence();
        double t = 0.0;
        const volatile double* pp = partials + (int64_t)m * gridDim.x;
        for (unsigned b = 0; b < gridDim.x; ++b) t += pp[b];
        t /= (double)p.d_inner;
        inv_out[m] = 1.0f / sqrtf((float)t + p.eps);
        counter[m] = 0;
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
template <typename Kern>
static int launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, const SgArgs& a) {
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

template <int KIND, int MT, int PRO, int EPI>
static int launch_sg_inst(const SgArgs& a, int grid, size_t smem) {
    auto kern = stream_gemv_kernel<KIND, MT, PRO, EPI>;
    static bool configured = false;
    if (!configured) {
        B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        configured = true;
    }
    return launch_pdl(kern, dim3(grid), dim3(SG_THREADS), smem, a);
}

static size_t sg_smem(const SgArgs& a, int mt) {
    return (size_t)SG_STAGES * a.stage_bytes + (size_t)mt * xs_floats(a.K) * 4 + 2 * SG_STAGES * 8 + 64;
}

template <int KIND, int PRO, int EPI>
static int launch_sg_mt(const SgArgs& a, int grid) {
    if (a.M == 1) return launch_sg_inst<KIND, 1, PRO, EPI>(a, grid, sg_smem(a, 1));
    if (a.M == 2) return launch_sg_inst<KIND, 2, PRO, EPI>(a, grid, sg_smem(a, 2));
    if (a.M <= 4) return launch_sg_inst<KIND, 4, PRO, EPI>(a, grid, sg_smem(a, 4));
    return launch_sg_inst<KIND, 8, PRO, EPI>(a, grid, sg_smem(a, 8));
}

// Fills the tiling fields and launches.  kind: template tag.
int stream_gemv(SgArgs a, int kind, int pro, int epi) {
    B200_REQUIRE(a.M >= 1 && a.M <= 8, "stream_gemv: 1..8 tokens per launch");
    B200_REQUIRE(a.K % 32 == 0 && (kind != 3 || a.K % 256 == 0), "stream_gemv: K not a multiple of the block size");
    a.row_bytes = row_bytes_of(kind, a.K);
    // rows per tile: ~8 KB, a multiple of what keeps every tile 16-byte aligned
    int align_rows = 1;
    while ((align_rows * a.row_bytes) % 16 != 0) align_rows *= 2;
    int R = (int)std::max<int64_t>(1, 8192 / a.row_bytes);
    R = std::max(align_rows, R / align_rows * align_rows);
    R = std::min(R, 64);
    if (R % align_rows) return fail(B200_EINVAL, "stream_gemv: row size %lld cannot be tiled to 16 bytes", (long long)a.row_bytes);
    a.rows_per_tile = R;
    a.num_tiles = ceil_div(a.N, R);
    a.stage_bytes = (int)((R * a.row_bytes + 127) / 128 * 128);
    a.status = stream_status_ptr();
    B200_REQUIRE(a.status, "stream_gemv: status word allocation failed");
    B200_REQUIRE((reinterpret_cast<uintptr_t>(a.w) & 15) == 0, "stream_gemv: weights must be 16-byte aligned");
    B200_REQUIRE(sg_smem(a, 8) <= 160 * 1024, "stream_gemv: K too large for the shared-memory staging");
    const int grid = std::min(a.num_tiles, 2 * num_sms());
#define SG_DISPATCH(KIND)                                                                               \
    if (pro == PRO_RMS && epi == EPI_STORE) return launch_sg_mt<KIND, PRO_RMS, EPI_STORE>(a, grid);     \
    if (pro == PRO_RMS && epi == EPI_INPROJ) return launch_sg_mt<KIND, PRO_RMS, EPI_INPROJ>(a, grid);   \
    if (pro == PRO_NONE && epi == EPI_RESIDUAL) return launch_sg_mt<KIND, PRO_NONE, EPI_RESIDUAL>(a, grid); \
    if (pro == PRO_NONE && epi == EPI_STORE) return launch_sg_mt<KIND, PRO_NONE, EPI_STORE>(a, grid);   \
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

int mamba_scan_norm(const float* bc, const float* dt_raw, const float* gate, const float* dt_bias,
                    const float* a_log, const float* D, const float* norm_w, float* ssm_state, float* u_out,
                    double* partials, unsigned* counter, float* inv_out, int batch, const MambaDims& p) {
    const int rows = p.n_heads * p.d_head;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ceil_div(rows, FS_WARPS), batch);
    cfg.blockDim = dim3(FS_WARPS * 32);
    cfg.stream = stream();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200_CUDA(cudaLaunchKernelEx(&cfg, mamba_scan_norm_kernel, bc, dt_raw, gate, dt_bias, a_log, D, norm_w, ssm_state,
                                 u_out, partials, counter, inv_out, p));
    ++g_kernel_launches;
    return B200_OK;
}

int mamba_scan_norm_blocks(const MambaDims& p) { return ceil_div(p.n_heads * p.d_head, FS_WARPS); }

}  // namespace b200
