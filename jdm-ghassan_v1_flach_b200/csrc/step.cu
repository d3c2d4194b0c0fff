// Whole-token decode step: the op sequence of Generator::decode_step_logits
// (inference/generator.cpp:221-443) and Generator::decode_mamba_layer (:456-617)
// for `batch` independent sequences, with per-sequence state (Mamba conv window and
// ssm state, paged fp16 KV cache) owned by the decoder, token ids and arg-max
// picks kept on the device, and no host synchronisation - so one step is a fixed
// list of kernels that is captured once into a CUDA graph and replayed.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

#include "fused.cuh"
#include "gemm.cuh"
#include "linear.cuh"
#include "persist.cuh"
#include "sampler.cuh"
#include "../../include/b200step.h"

namespace b200 {

// pos[b] = len[b]; len[b] += 1 : the position the new token is written at, and the
// number of cached tokens attention then sees.
__global__ void step_begin_kernel(int32_t* __restrict__ len, int32_t* __restrict__ pos, int batch) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < batch) { pos[b] = len[b]; len[b] += 1; }
}

// Store this token's K and V rows as fp16 into each sequence's page
// (the reference converts into its ring slot: generator.cpp:354-357).
__global__ void kv_append_kernel(const float* __restrict__ k, const float* __restrict__ v,
                                 uint16_t* __restrict__ k_pages, uint16_t* __restrict__ v_pages,
                                 const int32_t* __restrict__ page_table, const int32_t* __restrict__ pos,
                                 int max_pages, int page, int kvd) {
    const int b = blockIdx.y;
    const int p = pos[b];
    const int64_t row = (int64_t)page_table[(int64_t)b * max_pages + p / page] * page + p % page;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < kvd; c += gridDim.x * blockDim.x) {
        k_pages[row * kvd + c] = float_to_half_bits(k[(int64_t)b * kvd + c]);
        v_pages[row * kvd + c] = float_to_half_bits(v[(int64_t)b * kvd + c]);
    }
}

// out = a + s * b  (the reference's scale_inplace + add_inplace pair, generator.cpp:262-264)
__global__ void residual_kernel(float* __restrict__ x, const float* __restrict__ y, float s, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        x[i] = x[i] + y[i] * s;
}

// Row-wise greedy pick: largest finite logit, ties to the lowest id
// (core/math_cpu.cpp:709-722).  One block per sequence.
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float* __restrict__ logits, int V,
                                                           int32_t* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* row = logits + (int64_t)blockIdx.x * V;
    float bv = 0.0f;
    int bi = -1;
    auto visit = [&](float v, int i) {
        if (isfinite(v) && (bi < 0 || v > bv)) { bv = v; bi = i; }   // ascending i per thread
    };
    if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        // four runs of four per pass, all loads issued before the first compare
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int n4 = V >> 2;
        for (int q0 = threadIdx.x; q0 < n4; q0 += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * blockDim.x;
                v[u] = q < n4 ? row4[q] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * blockDim.x;
                if (q < n4) {
                    visit(v[u].x, 4 * q);
                    visit(v[u].y, 4 * q + 1);
                    visit(v[u].z, 4 * q + 2);
                    visit(v[u].w, 4 * q + 3);
                }
            }
        }
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) visit(row[i], i);
    }
    auto take = [&](float ov, int oi) {
        if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) take(__shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { sv[wid] = bv; si[wid] = bi; }
    __syncthreads();
    if (wid == 0) {
        bv = sv[lane];
        bi = si[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) take(__shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (lane == 0) {
            if (bi < 0) {   // nothing finite: the reference's serial fallback
                bi = 0;
                for (int i = 1; i < V; ++i) if (row[i] > row[bi]) bi = i;
            }
            out[blockIdx.x] = bi;
        }
    }
}

struct LayerW {
    const float *attn_norm = nullptr, *ffn_norm = nullptr;
    const void *mamba_in = nullptr, *mamba_out = nullptr;
    const float *conv_w = nullptr, *conv_b = nullptr, *dt_bias = nullptr, *a_log = nullptr, *D = nullptr, *mamba_norm = nullptr;
    const void *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr;
    const float *router = nullptr, *router_bias = nullptr;
    const void *gate = nullptr, *up = nullptr, *down = nullptr, *sh_gate = nullptr, *sh_up = nullptr, *sh_down = nullptr;
    // state
    float *conv_state = nullptr, *ssm_state = nullptr;       // Mamba layers
    uint16_t *k_pages = nullptr, *v_pages = nullptr;         // attention layers
};

}  // namespace b200

using namespace b200;

struct b200_decoder {
    int batch, vocab, d, n_layers;
    std::vector<int> types;
    int H, KV, hd, rope_type;
    int mh, mdh, mds, mk, d_inner, conv_dim;
    int ne, K, E, SH;
    int max_ctx, page, max_pages, qkind;
    float eps, emb_mult, res_mult, attn_scale, logits_scaling;
    const uint16_t *embed = nullptr, *lm_head = nullptr;
    const float *final_norm = nullptr, *inv_freq = nullptr;
    std::vector<LayerW> L;
    // buffers
    std::vector<void*> owned;
    __half* xb16 = nullptr;      // xb once more as fp16 rows (per-op step with enough rows for the GEMMs)
    float *x = nullptr, *xb = nullptr, *proj = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr, *logits = nullptr;
    int32_t *tok = nullptr, *next = nullptr, *len = nullptr, *pos = nullptr, *page_table = nullptr;
    int position = 0;
    int fused = 0, use_graph = 0;
    int rope_refresh_as_reference = 0;
    cudaGraphExec_t graph = nullptr;
    const int32_t* graph_tok = nullptr;
    int32_t* graph_next = nullptr;
    cudaStream_t own_stream = nullptr;
    int launches = 0;
    int32_t *h_tok = nullptr, *h_next = nullptr;   // pinned staging for the host entry point
    // fused mode scratch
    float *f_gate = nullptr, *f_bc = nullptr, *f_dt = nullptr, *f_u = nullptr;
    double* f_partials = nullptr;
    int f_blocks = 0;
    float *f_logits = nullptr, *f_w = nullptr, *f_act = nullptr, *f_shact = nullptr;
    int32_t* f_idx = nullptr;
    // persistent mode (fused == 2, batch 1): device copies of the layer table and the phase
    // list, the launch arguments, and the runs of phases between attention layers
    PArgs pa;
    PLayer* p_layers = nullptr;
    POp* p_ops = nullptr;
    struct Segment { int op_begin, op_end, attn_layer; };
    std::vector<Segment> segments;
    bool p_ready = false;
    unsigned long long* pa_bar = nullptr;
    unsigned int *pa_done = nullptr, *pa_flag = nullptr, *pa_rt = nullptr;
    float *pa_bcd = nullptr, *pa_shout = nullptr;
    double* pa_partials = nullptr;
    unsigned long long* pa_trace = nullptr;
    unsigned int test_spin_limit = 0;          // test hook (b200_decoder_test_barrier)
    int test_skip_cta = -1;
    unsigned long long ws_generation = 0;      // workspace generation the captured graph was recorded at
    // sampling (b200_decoder_set_sampling): per-sequence history ring, pushed-token counts and
    // generator streams, all on the device; scratch of the selection kernels
    bool sampling = false;
    b200_sampling samp{};
    int32_t *hist = nullptr, *hist_total = nullptr;
    uint64_t* rng = nullptr;
    void* samp_ws = nullptr;
    size_t samp_ws_bytes = 0;
};
constexpr int DEC_HIST_CAP = 8192;             // Generator::HIST_MAX, inference/generator.h:96

// RoPE is applied unless the decoder mirrors the reference Generator's handling of the
// position word (b200_decoder_set_rope_refresh) on a model whose first layer is a Mamba layer.
static bool rope_on(const b200_decoder* dec) {
    return dec->rope_type >= 0 && !(dec->rope_refresh_as_reference && !dec->types.empty() && dec->types[0] == 0);
}

static int dev_alloc(b200_decoder* dec, void** p, size_t bytes) {
    B200_CUDA(cudaMalloc(p, bytes ? bytes : 4));
    B200_CUDA(cudaMemset(*p, 0, bytes ? bytes : 4));
    dec->owned.push_back(*p);
    return B200_OK;
}

static void drop_graph(b200_decoder* dec) {
    if (dec->graph) cudaGraphExecDestroy(dec->graph);
    dec->graph = nullptr;
}

// The next token of sequences [b0, b0 + B) from their logits: the greedy arg-max, or - with
// b200_decoder_set_sampling - Sampler::sample on the device after the T tokens just fed
// (fed [B, T]) have joined the sequences' histories.  next == nullptr only records the history.
static int pick_next(b200_decoder* dec, float* logits, const int32_t* fed, int T, int32_t* next, int b0, int B,
                     const int32_t* seq_off = nullptr) {
    if (!dec->sampling) {
        if (!next) return B200_OK;
        argmax_rows_kernel<<<B, 1024, 0, stream()>>>(logits, dec->vocab, next);
        B200_LAUNCH_CHECK("argmax_rows_kernel");
        return B200_OK;
    }
    int32_t* hist = dec->hist + (int64_t)b0 * DEC_HIST_CAP;
    int rc = history_push_prompt(hist, DEC_HIST_CAP, dec->hist_total + b0, fed, B, T, seq_off);
    if (rc || !next) return rc;
    return sample_rows(logits, dec->vocab, B, hist, DEC_HIST_CAP, dec->hist_total + b0, dec->samp, dec->rng + 4 * b0, next,
                       dec->samp_ws);
}

// The op sequence of one token, enqueued on the library's current stream.
constexpr int RRN_PER = 16;      // row elements a thread keeps in registers: dim <= 4096
__global__ void residual_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ y, float s,
                                        const float* __restrict__ w, float* __restrict__ out, int dim, float eps,
                                        __half* __restrict__ out16);

static int enqueue_step(b200_decoder* dec, const int32_t* tokens, int32_t* next) {
    const int B = dec->batch, d = dec->d;
    cudaStream_t st = stream();
    int rc;
#define STEP(call)              \
    do {                        \
        rc = (call);            \
        if (rc) return rc;      \
    } while (0)
    step_begin_kernel<<<ceil_div(B, 128), 128, 0, st>>>(dec->len, dec->pos, B);
    B200_LAUNCH_CHECK("step_begin_kernel");
    STEP(b200_embedding_forward_half(tokens, dec->embed, dec->x, B, d, dec->vocab));
    if (dec->emb_mult != 1.0f) STEP(b200_scale_inplace(dec->x, dec->emb_mult, (int64_t)B * d));
    const int res_grid = std::min(ceil_div(B * d, 256), num_sms() * 8);
    // x += res_mult * proj followed by the next norm, one launch when the row fits the registers
    // With enough rows for the tensor-core GEMMs the norm also leaves its rows as fp16 and registers
    // them, so the projections that read xb next (in_proj; q, k, v; the shared expert) skip their
    // conversion pass; the entry is dropped before xb is written again and when the step ends.
    const bool rows16 = B >= GEMM_MIN_ROWS && d % 8 == 0;
    f16_shadow_clear();
    auto residual_norm = [&](const float* norm_w) -> int {
        f16_shadow_clear();
        if (d <= RRN_PER * 256) {
            residual_rmsnorm_kernel<<<(unsigned)B, 256, 0, st>>>(dec->x, dec->proj, dec->res_mult, norm_w, dec->xb, d,
                                                                dec->eps, rows16 ? dec->xb16 : nullptr);
            B200_LAUNCH_CHECK("residual_rmsnorm_kernel");
            if (rows16) f16_shadow_set(dec->xb, dec->xb16, B, d);
            return B200_OK;
        }
        residual_kernel<<<res_grid, 256, 0, st>>>(dec->x, dec->proj, dec->res_mult, (int64_t)B * d);
        B200_LAUNCH_CHECK("residual_kernel");
        return b200_rmsnorm_forward(dec->x, norm_w, dec->xb, nullptr, B, d, dec->eps);
    };
    if (dec->n_layers > 0) STEP(b200_rmsnorm_forward(dec->x, dec->L[0].attn_norm, dec->xb, nullptr, B, d, dec->eps));
    else STEP(b200_rmsnorm_forward(dec->x, dec->final_norm, dec->xb, nullptr, B, d, dec->eps));
    for (int l = 0; l < dec->n_layers; ++l) {
        LayerW& w = dec->L[l];
        if (dec->types[l] == 0) {
            STEP(b200_mamba2_step_batched(dec->xb, static_cast<const uint16_t*>(w.mamba_in), w.conv_w, w.conv_b,
                                          w.dt_bias, w.a_log, w.D, w.mamba_norm,
                                          static_cast<const uint16_t*>(w.mamba_out), w.conv_state, w.ssm_state,
                                          dec->proj, B, d, dec->d_inner, dec->conv_dim, dec->mh, dec->mdh, dec->mds,
                                          dec->mk, dec->eps, dec->qkind));
        } else {
            const int qd = dec->H * dec->hd, kvd = dec->KV * dec->hd;
            if (dec->qkind >= 0) {
                STEP(b200_linear_forward_q4(dec->xb, static_cast<const uint16_t*>(w.wq), dec->q, B, d, qd, dec->qkind));
                STEP(b200_linear_forward_q4(dec->xb, static_cast<const uint16_t*>(w.wk), dec->k, B, d, kvd, dec->qkind));
                STEP(b200_linear_forward_q4(dec->xb, static_cast<const uint16_t*>(w.wv), dec->v, B, d, kvd, dec->qkind));
            } else {
                STEP(b200_linear_forward_fp16(dec->xb, static_cast<const uint16_t*>(w.wq), dec->q, B, d, qd));
                STEP(b200_linear_forward_fp16(dec->xb, static_cast<const uint16_t*>(w.wk), dec->k, B, d, kvd));
                STEP(b200_linear_forward_fp16(dec->xb, static_cast<const uint16_t*>(w.wv), dec->v, B, d, kvd));
            }
            if (rope_on(dec))
                STEP(b200_rope_forward_cached(dec->q, dec->k, dec->pos, dec->inv_freq, B, dec->H, dec->KV, dec->hd,
                                              dec->rope_type));
            kv_append_kernel<<<dim3(ceil_div(kvd, 256), B), 256, 0, st>>>(dec->k, dec->v, w.k_pages, w.v_pages,
                                                                         dec->page_table, dec->pos, dec->max_pages,
                                                                         dec->page, kvd);
            B200_LAUNCH_CHECK("kv_append_kernel");
            STEP(b200_attention_decode_paged_fp16(dec->q, w.k_pages, w.v_pages, dec->page_table, dec->len, dec->attn,
                                                  B, dec->max_pages, dec->page, dec->H, dec->KV, dec->hd,
                                                  dec->attn_scale));
            if (dec->qkind >= 0)
                STEP(b200_linear_forward_q4(dec->attn, static_cast<const uint16_t*>(w.wo), dec->proj, B, qd, d, dec->qkind));
            else
                STEP(b200_linear_forward_fp16(dec->attn, static_cast<const uint16_t*>(w.wo), dec->proj, B, qd, d));
        }
        STEP(residual_norm(w.ffn_norm));
        STEP(b200_moe_forward_bias_half(dec->xb, w.router, w.router_bias, static_cast<const uint16_t*>(w.gate),
                                        static_cast<const uint16_t*>(w.up), static_cast<const uint16_t*>(w.down),
                                        static_cast<const uint16_t*>(w.sh_gate), static_cast<const uint16_t*>(w.sh_up),
                                        static_cast<const uint16_t*>(w.sh_down), dec->proj, nullptr, nullptr, nullptr,
                                        nullptr, nullptr, nullptr, B, d, dec->E, dec->ne, dec->K, dec->SH, dec->qkind));
        STEP(residual_norm(l + 1 < dec->n_layers ? dec->L[l + 1].attn_norm : dec->final_norm));
    }
    rc = b200_linear_forward_fp16(dec->xb, dec->lm_head, dec->logits, B, d, dec->vocab);
    f16_shadow_clear();
    if (rc) return rc;
    if (dec->logits_scaling != 1.0f)
        STEP(b200_scale_inplace(dec->logits, 1.0f / dec->logits_scaling, (int64_t)B * dec->vocab));
    STEP(pick_next(dec, dec->logits, tokens, 1, next, 0, B));
#undef STEP
    return B200_OK;
}

// Fused variant (batch <= 8): the RMSNorm before each projection runs as that
// projection's prologue, the residual add as the epilogue of the layer's last
// projection, the Mamba conv step inside in_proj's epilogue and the gated norm is
// folded into the state update + out_proj.  Kernels are chained with programmatic
// dependent launch so each one streams its weights while its predecessor drains.
// dry = true walks the same calls but only validates shapes and tiling (no launch).
static int enqueue_step_fused(b200_decoder* dec, const int32_t* tokens, int32_t* next, bool dry = false) {
    const int B = dec->batch, d = dec->d;
    cudaStream_t st = stream();
    const int kind = tag_of_qkind(dec->qkind);
    int rc;
#define STEP(call)              \
    do {                        \
        rc = (call);            \
        if (rc) return rc;      \
    } while (0)
    if (!dry) {
        step_begin_kernel<<<ceil_div(B, 128), 128, 0, st>>>(dec->len, dec->pos, B);
        B200_LAUNCH_CHECK("step_begin_kernel");
        STEP(b200_embedding_forward_half(tokens, dec->embed, dec->x, B, d, dec->vocab));
        if (dec->emb_mult != 1.0f) STEP(b200_scale_inplace(dec->x, dec->emb_mult, (int64_t)B * d));
    }
    const int res_grid = std::min(ceil_div(B * d, 256), num_sms() * 8);
    MambaDims p;
    p.d = d; p.d_inner = dec->d_inner; p.conv_dim = dec->conv_dim; p.n_heads = dec->mh; p.d_head = dec->mdh;
    p.d_state = dec->mds; p.k = dec->mk; p.eps = dec->eps; p.proj = dec->d_inner + dec->conv_dim + dec->mh;
    auto base = [&](const void* w, int N, int K, const float* x, int xs) {
        SgArgs a;
        a.w = static_cast<const uint8_t*>(w); a.N = N; a.K = K; a.M = B; a.x = x; a.x_stride = xs; a.eps = dec->eps;
        a.dry = dry;
        return a;
    };
    for (int l = 0; l < dec->n_layers; ++l) {
        LayerW& w = dec->L[l];
        if (dec->types[l] == 0) {
            SgArgs a = base(w.mamba_in, p.proj, d, dec->x, d);
            a.norm_w = w.attn_norm; a.p = p; a.conv_w = w.conv_w; a.conv_b = w.conv_b; a.conv_state = w.conv_state;
            a.gate = dec->f_gate; a.bc = dec->f_bc; a.dt_raw = dec->f_dt;
            STEP(stream_gemv(a, kind, PRO_RMS, EPI_INPROJ));
            if (!dry)
                STEP(mamba_scan_norm(dec->f_bc, dec->f_dt, dec->f_gate, w.dt_bias, w.a_log, w.D, w.mamba_norm,
                                     w.ssm_state, dec->f_u, dec->f_partials, B, p));
            SgArgs c = base(w.mamba_out, d, dec->d_inner, dec->f_u, dec->d_inner);
            c.in_partials = dec->f_partials; c.n_partials = dec->f_blocks; c.in_dim = dec->d_inner;
            c.resid = dec->x; c.y_stride = d; c.res_mult = dec->res_mult;
            STEP(stream_gemv(c, kind, PRO_NONE, EPI_RESIDUAL));
        } else {
            const int qd = dec->H * dec->hd, kvd = dec->KV * dec->hd;
            // q, k and v in one launch: one norm, one staging of the activations
            SgArgs aq = base(w.wq, qd, d, dec->x, d);
            aq.norm_w = w.attn_norm; aq.y = dec->q; aq.y_stride = qd;
            aq.w2 = static_cast<const uint8_t*>(w.wk); aq.N2 = kvd; aq.y2 = dec->k; aq.y2_stride = kvd;
            aq.w3 = static_cast<const uint8_t*>(w.wv); aq.N3 = kvd; aq.y3 = dec->v; aq.y3_stride = kvd;
            STEP(stream_gemv(aq, kind, PRO_RMS, EPI_STORE));
            if (!dry) {
                if (rope_on(dec))
                    STEP(b200_rope_forward_cached(dec->q, dec->k, dec->pos, dec->inv_freq, B, dec->H, dec->KV, dec->hd,
                                                  dec->rope_type));
                kv_append_kernel<<<dim3(ceil_div(kvd, 256), B), 256, 0, st>>>(dec->k, dec->v, w.k_pages, w.v_pages,
                                                                             dec->page_table, dec->pos,
                                                                             dec->max_pages, dec->page, kvd);
                B200_LAUNCH_CHECK("kv_append_kernel");
                STEP(b200_attention_decode_paged_fp16(dec->q, w.k_pages, w.v_pages, dec->page_table, dec->len,
                                                      dec->attn, B, dec->max_pages, dec->page, dec->H, dec->KV,
                                                      dec->hd, dec->attn_scale));
            }
            SgArgs ao = base(w.wo, d, qd, dec->attn, qd);
            ao.resid = dec->x; ao.y_stride = d; ao.res_mult = dec->res_mult;
            STEP(stream_gemv(ao, kind, PRO_NONE, EPI_RESIDUAL));
        }
        MoeFusedArgs mo;
        mo.x = dec->x; mo.norm_w = w.ffn_norm; mo.eps = dec->eps; mo.router_w = w.router; mo.router_bias = w.router_bias;
        mo.gates = static_cast<const uint8_t*>(w.gate); mo.ups = static_cast<const uint8_t*>(w.up);
        mo.downs = static_cast<const uint8_t*>(w.down); mo.sh_g = static_cast<const uint8_t*>(w.sh_gate);
        mo.sh_u = static_cast<const uint8_t*>(w.sh_up); mo.sh_d = static_cast<const uint8_t*>(w.sh_down);
        mo.logits = dec->f_logits; mo.idx = dec->f_idx; mo.w = dec->f_w; mo.act = dec->f_act; mo.sh_act = dec->f_shact;
        mo.resid = dec->x; mo.res_mult = dec->res_mult;
        mo.M = B; mo.d = d; mo.E = dec->E; mo.ne = dec->ne; mo.K = dec->K;
        mo.SH = (dry || (w.sh_gate && w.sh_up && w.sh_down)) ? dec->SH : 0;
        mo.dry = dry;
        STEP(moe_fused(mo, kind));
    }
    SgArgs h = base(dec->lm_head, dec->vocab, d, dec->x, d);
    h.norm_w = dec->final_norm; h.y = dec->logits; h.y_stride = dec->vocab; h.out_scale = 1.0f / dec->logits_scaling;
    STEP(stream_gemv(h, KIND_F16, PRO_RMS, EPI_STORE));
    if (dry) return B200_OK;
    STEP(pick_next(dec, dec->logits, tokens, 1, next, 0, B));
#undef STEP
    return B200_OK;
}

// ---------------------------------------------------------------------------
// Prompt processing: T tokens of every sequence at once through the many-token
// kernels (tensor-core GEMMs, chunked SSD scan, tensor-core attention, grouped MoE),
// leaving the per-sequence state exactly where T decode steps would have left it:
// ssm state, convolution window, KV pages, lengths.
// ---------------------------------------------------------------------------
constexpr int PREFILL_GROUP_TOKENS = 32768;
__global__ void prefill_pos_kernel(int32_t* __restrict__ pos, int B, int T) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < B * T) pos[i] = i % T;
}
__global__ void prefill_len_kernel(int32_t* __restrict__ len, int32_t* __restrict__ pos, int B, int T) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) { len[b] = T; pos[b] = T - 1; }
}
// k, v [B, T, kvd] fp32 -> fp16 rows of the sequences' pages
__global__ void kv_prefill_kernel(const float* __restrict__ k, const float* __restrict__ v, uint16_t* __restrict__ k_pages,
                                  uint16_t* __restrict__ v_pages, const int32_t* __restrict__ page_table, int T,
                                  int max_pages, int page, int kvd) {
    const int t = blockIdx.y, b = blockIdx.z;
    const int64_t row = (int64_t)page_table[(int64_t)b * max_pages + t / page] * page + t % page;
    const int64_t src = ((int64_t)b * T + t) * kvd;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < kvd; c += gridDim.x * blockDim.x) {
        k_pages[row * kvd + c] = float_to_half_bits(k[src + c]);
        v_pages[row * kvd + c] = float_to_half_bits(v[src + c]);
    }
}
// The same for packed sequences: row r belongs to sequence seq[r] at position pos[r].
__global__ void kv_prefill_packed_kernel(const float* __restrict__ k, const float* __restrict__ v,
                                         uint16_t* __restrict__ k_pages, uint16_t* __restrict__ v_pages,
                                         const int32_t* __restrict__ page_table, const int32_t* __restrict__ seq,
                                         const int32_t* __restrict__ pos, int max_pages, int page, int kvd) {
    const int64_t r = blockIdx.y;
    const int b = seq[r], t = pos[r];
    const int64_t row = (int64_t)page_table[(int64_t)b * max_pages + t / page] * page + t % page;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < kvd; c += gridDim.x * blockDim.x) {
        k_pages[row * kvd + c] = float_to_half_bits(k[r * kvd + c]);
        v_pages[row * kvd + c] = float_to_half_bits(v[r * kvd + c]);
    }
}
// dst[b, :] = src[last row of sequence b, :]; len[b], pos[b] from the sequence's length
__global__ void last_rows_packed_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                        const int32_t* __restrict__ seq_off, int B, int d) {
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < (int64_t)B * d) {
        const int b = (int)(i / d), c = (int)(i - (int64_t)b * d);
        dst[i] = src[(int64_t)(seq_off[b + 1] - 1) * d + c];
    }
}
__global__ void prefill_len_packed_kernel(int32_t* __restrict__ len, int32_t* __restrict__ pos,
                                          const int32_t* __restrict__ seq_off, int B) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) {
        const int n = seq_off[b + 1] - seq_off[b];
        len[b] = n;
        pos[b] = n - 1;
    }
}
// dst[b, :] = src[b, T-1, :]
__global__ void last_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int B, int T, int d) {
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < (int64_t)B * d) {
        const int b = (int)(i / d), c = (int)(i - (int64_t)b * d);
        dst[i] = src[((int64_t)b * T + T - 1) * d + c];
    }
}

// x = x + s * y, then out = rmsnorm(x) * w: the residual update and the norm that follows it
// in one pass over the row (the same operations in the same order as residual_kernel and
// rmsnorm_kernel: double sum of squares, inv rounded to float).  One block per row.
// out16 (optional): the normalised row once more as fp16 (clamped), for the tensor-core GEMMs.
__global__ void __launch_bounds__(256) residual_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ y, float s,
                                                               const float* __restrict__ w, float* __restrict__ out,
                                                               int dim, float eps, __half* __restrict__ out16) {
    __shared__ double red[32];
    const int64_t r = blockIdx.x;
    float* xr = x + r * dim;
    const float* yr = y + r * dim;
    float v[RRN_PER];
    double ss = 0.0;
#pragma unroll
    for (int j = 0; j < RRN_PER; ++j) {
        const int i = j * 256 + threadIdx.x;
        v[j] = 0.0f;
        if (i < dim) {
            v[j] = xr[i] + yr[i] * s;
            xr[i] = v[j];
            ss += (double)v[j] * (double)v[j];
        }
    }
    ss = block_sum_d(ss, red);
    const double inv_d = 1.0 / sqrt(ss / (double)dim + (double)eps);
    const float inv = isfinite(inv_d) ? (float)inv_d : 0.0f;
    float* o = out + r * dim;
#pragma unroll
    for (int j = 0; j < RRN_PER; ++j) {
        const int i = j * 256 + threadIdx.x;
        if (i < dim) {
            const float r2 = v[j] * inv * w[i];
            o[i] = r2;
            if (out16) out16[r * dim + i] = __float2half_rn(fminf(fmaxf(r2, -65504.0f), 65504.0f));
        }
    }
}

// Sequences [b0, b0 + B) of the decoder; tokens / next point at that group's first sequence.
// score_targets (device, [B * T], optional): instead of the last token's logits, every row's
// cross-entropy against its target is added to score_acc (cross_entropy_accumulate), the
// lm_head running over SCORE_ROWS rows at a time.
constexpr int SCORE_ROWS = 512;
// lay (optional): the B sequences have different lengths and their tokens lie packed back to
// back as lay describes; T is then ignored.
static int prefill(b200_decoder* dec, const int32_t* tokens, int T, int32_t* next, int b0, int B,
                   const int32_t* score_targets = nullptr, double* score_acc = nullptr, const SeqLayout* lay = nullptr) {
    NvtxRange range(score_targets ? "b200.score_tokens" : lay ? "b200.prefill_ragged" : "b200.prefill");
    const int d = dec->d;
    float *dx = dec->x + (int64_t)b0 * d, *dxb = dec->xb + (int64_t)b0 * d, *dlogits = dec->logits + (int64_t)b0 * dec->vocab;
    const int32_t* page_table = dec->page_table + (int64_t)b0 * dec->max_pages;
    const int64_t NT = lay ? lay->rows : (int64_t)B * T;
    const int qd = dec->H * dec->hd, kvd = dec->KV * dec->hd;
    cudaStream_t st = stream();
    int rc;
#define STEP(call)              \
    do {                        \
        rc = (call);            \
        if (rc) return rc;      \
    } while (0)
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off += (bytes + 255) & ~(size_t)255; return o; };
    const size_t o_x = take(NT * d * 4), o_xb = take(NT * d * 4), o_y = take(NT * d * 4), o_q = take(NT * qd * 4),
                 o_k = take(NT * kvd * 4), o_v = take(NT * kvd * 4), o_at = take(NT * qd * 4), o_pos = take(NT * 4),
                 o_xb16 = take(NT * d * 2);
    void* wsp;
    STEP(workspace(WS_PREFILL).ensure(off + 256, &wsp));
    char* base = static_cast<char*>(wsp);
    float *x = reinterpret_cast<float*>(base + o_x), *xb = reinterpret_cast<float*>(base + o_xb),
          *y = reinterpret_cast<float*>(base + o_y), *q = reinterpret_cast<float*>(base + o_q),
          *k = reinterpret_cast<float*>(base + o_k), *v = reinterpret_cast<float*>(base + o_v),
          *at = reinterpret_cast<float*>(base + o_at);
    const int32_t* pos = lay ? lay->pos : reinterpret_cast<int32_t*>(base + o_pos);
    __half* xb16 = reinterpret_cast<__half*>(base + o_xb16);      // fp16 copy of xb for the GEMMs (when d % 8 == 0)
    const bool want16 = d % 8 == 0 && d <= RRN_PER * 256;
    const int kind = tag_of_qkind(dec->qkind);
    MambaDims p;
    p.d = d; p.d_inner = dec->d_inner; p.conv_dim = dec->conv_dim; p.n_heads = dec->mh; p.d_head = dec->mdh;
    p.d_state = dec->mds; p.k = dec->mk; p.eps = dec->eps; p.proj = dec->d_inner + dec->conv_dim + dec->mh;
    auto lin = [&](const float* in, const void* w, float* out, int K, int N, const __half* in16 = nullptr) {
        if (in16 && linear_uses_gemm(w, kind, out, (int)NT, K, N)) return linear_a16(in16, w, kind, out, (int)NT, K, N);
        return dec->qkind >= 0 ? b200_linear_forward_q4(in, static_cast<const uint16_t*>(w), out, (int)NT, K, N, dec->qkind)
                               : b200_linear_forward_fp16(in, static_cast<const uint16_t*>(w), out, (int)NT, K, N);
    };
    const int res_grid = (int)std::min<int64_t>(ceil_div64(NT * d, 256), (int64_t)num_sms() * 16);
    STEP(b200_embedding_forward_half(tokens, dec->embed, x, NT, d, dec->vocab));
    if (dec->emb_mult != 1.0f) STEP(b200_scale_inplace(x, dec->emb_mult, NT * d));
    if (rope_on(dec) && !lay) {
        prefill_pos_kernel<<<(unsigned)ceil_div64(NT, 256), 256, 0, st>>>(reinterpret_cast<int32_t*>(base + o_pos), B, T);
        B200_LAUNCH_CHECK("prefill_pos_kernel");
    }
    // x += res_mult * y followed by the next norm; fused when the row fits the registers
    auto residual_norm = [&](const float* norm_w) -> int {
        if (norm_w && d <= RRN_PER * 256) {
            residual_rmsnorm_kernel<<<(unsigned)NT, 256, 0, st>>>(x, y, dec->res_mult, norm_w, xb, d, dec->eps,
                                                                  want16 ? xb16 : nullptr);
            B200_LAUNCH_CHECK("residual_rmsnorm_kernel");
            return B200_OK;
        }
        residual_kernel<<<res_grid, 256, 0, st>>>(x, y, dec->res_mult, NT * d);
        B200_LAUNCH_CHECK("residual_kernel");
        return norm_w ? b200_rmsnorm_forward(x, norm_w, xb, nullptr, NT, d, dec->eps) : B200_OK;
    };
    if (dec->n_layers > 0) {
        STEP(b200_rmsnorm_forward(x, dec->L[0].attn_norm, xb, nullptr, NT, d, dec->eps));
        if (want16) STEP(pack_rows_f16(xb, nullptr, 1, xb16, NT, d));
    }
    for (int l = 0; l < dec->n_layers; ++l) {
        LayerW& w = dec->L[l];
        NvtxRange layer_range(dec->types[l] == 0 ? "b200.prefill.mamba+moe" : "b200.prefill.attention+moe");
        if (dec->types[l] == 0) {
            STEP(mamba2_forward(xb, w.mamba_in, w.conv_w, w.conv_b, w.dt_bias, w.a_log, w.D, w.mamba_norm, w.mamba_out,
                                w.ssm_state + (int64_t)b0 * dec->d_inner * dec->mds, y, B, T, p, kind,
                                w.conv_state + (int64_t)b0 * dec->conv_dim * std::max(dec->mk - 1, 1),
                                want16 ? xb16 : nullptr, lay));
        } else {
            STEP(lin(xb, w.wq, q, d, qd, want16 ? xb16 : nullptr));
            STEP(lin(xb, w.wk, k, d, kvd, want16 ? xb16 : nullptr));
            STEP(lin(xb, w.wv, v, d, kvd, want16 ? xb16 : nullptr));
            if (rope_on(dec))
                STEP(b200_rope_forward_cached(q, k, pos, dec->inv_freq, NT, dec->H, dec->KV, dec->hd, dec->rope_type));
            if (!lay) {
                kv_prefill_kernel<<<dim3(ceil_div(kvd, 256), T, B), 256, 0, st>>>(k, v, w.k_pages, w.v_pages, page_table, T,
                                                                                dec->max_pages, dec->page, kvd);
                B200_LAUNCH_CHECK("kv_prefill_kernel");
                STEP(b200_attention_forward_ex(q, k, v, at, nullptr, B, T, dec->H, dec->KV, dec->hd, dec->attn_scale, 0, nullptr));
            } else {
                kv_prefill_packed_kernel<<<dim3(ceil_div(kvd, 256), (unsigned)NT), 256, 0, st>>>(
                    k, v, w.k_pages, w.v_pages, page_table, lay->seq, lay->pos, dec->max_pages, dec->page, kvd);
                B200_LAUNCH_CHECK("kv_prefill_packed_kernel");
                // causal attention inside each sequence: one call per sequence on its rows
                for (int b = 0; b < B; ++b) {
                    const int64_t r0 = lay->host_off[b];
                    STEP(b200_attention_forward_ex(q + r0 * qd, k + r0 * kvd, v + r0 * kvd, at + r0 * qd, nullptr, 1,
                                                   lay->host_off[b + 1] - lay->host_off[b], dec->H, dec->KV, dec->hd,
                                                   dec->attn_scale, 0, nullptr));
                }
            }
            STEP(lin(at, w.wo, y, qd, d));
        }
        STEP(residual_norm(w.ffn_norm));
        STEP(b200_moe_forward_bias_half(xb, w.router, w.router_bias, static_cast<const uint16_t*>(w.gate),
                                        static_cast<const uint16_t*>(w.up), static_cast<const uint16_t*>(w.down),
                                        static_cast<const uint16_t*>(w.sh_gate), static_cast<const uint16_t*>(w.sh_up),
                                        static_cast<const uint16_t*>(w.sh_down), y, nullptr, nullptr, nullptr, nullptr,
                                        nullptr, nullptr, NT, d, dec->E, dec->ne, dec->K, dec->SH, dec->qkind));
        STEP(residual_norm(l + 1 < dec->n_layers ? dec->L[l + 1].attn_norm : nullptr));
    }
    if (score_targets) {
        const int V = dec->vocab;
        const int rows_max = (int)std::min<int64_t>(SCORE_ROWS, NT);
        void* sws;
        STEP(workspace(WS_SAMPLE).ensure(256 + (size_t)rows_max * 8 + 256 + (size_t)rows_max * V * 4, &sws));
        double* losses = reinterpret_cast<double*>(static_cast<char*>(sws) + 256);
        float* lg = reinterpret_cast<float*>(static_cast<char*>(sws) + 256 + (((size_t)rows_max * 8 + 255) & ~(size_t)255));
        for (int64_t r0 = 0; r0 < NT; r0 += SCORE_ROWS) {
            const int rows = (int)std::min<int64_t>(SCORE_ROWS, NT - r0);
            STEP(b200_rmsnorm_forward(x + r0 * d, dec->final_norm, xb + r0 * d, nullptr, rows, d, dec->eps));
            STEP(b200_linear_forward_fp16(xb + r0 * d, dec->lm_head, lg, rows, d, V));
            if (dec->logits_scaling != 1.0f) STEP(b200_scale_inplace(lg, 1.0f / dec->logits_scaling, (int64_t)rows * V));
            STEP(cross_entropy_accumulate(lg, score_targets + r0, rows, V, 0.0f, losses, score_acc));
        }
        STEP(pick_next(dec, nullptr, tokens, T, nullptr, b0, B, lay ? lay->seq_off : nullptr));
    } else {
        // logits of the last token of every sequence
        if (lay) last_rows_packed_kernel<<<(unsigned)ceil_div64((int64_t)B * d, 256), 256, 0, st>>>(x, dx, lay->seq_off, B, d);
        else last_rows_kernel<<<(unsigned)ceil_div64((int64_t)B * d, 256), 256, 0, st>>>(x, dx, B, T, d);
        B200_LAUNCH_CHECK("last_rows_kernel");
        STEP(b200_rmsnorm_forward(dx, dec->final_norm, dxb, nullptr, B, d, dec->eps));
        STEP(b200_linear_forward_fp16(dxb, dec->lm_head, dlogits, B, d, dec->vocab));
        if (dec->logits_scaling != 1.0f)
            STEP(b200_scale_inplace(dlogits, 1.0f / dec->logits_scaling, (int64_t)B * dec->vocab));
        STEP(pick_next(dec, dlogits, tokens, T, next, b0, B, lay ? lay->seq_off : nullptr));
    }
    if (lay) prefill_len_packed_kernel<<<ceil_div(B, 128), 128, 0, st>>>(dec->len + b0, dec->pos + b0, lay->seq_off, B);
    else prefill_len_kernel<<<ceil_div(B, 128), 128, 0, st>>>(dec->len + b0, dec->pos + b0, B, T);
    B200_LAUNCH_CHECK("prefill_len_kernel");
#undef STEP
    return B200_OK;
}

static int check_ready(const b200_decoder* dec);

// The attention mixer of one layer on the fused few-token kernels (shared by the fused and
// the persistent modes): q/k/v in one launch with the norm as prologue, RoPE, K/V append,
// split-KV attention, output projection with the residual add as epilogue.
static int enqueue_attention_fused(b200_decoder* dec, LayerW& w, int kind, bool dry) {
    const int B = dec->batch, d = dec->d;
    cudaStream_t st = stream();
    const int qd = dec->H * dec->hd, kvd = dec->KV * dec->hd;
    int rc;
    auto base = [&](const void* wt, int N, int K, const float* x, int xs) {
        SgArgs a;
        a.w = static_cast<const uint8_t*>(wt); a.N = N; a.K = K; a.M = B; a.x = x; a.x_stride = xs; a.eps = dec->eps;
        a.dry = dry;
        return a;
    };
    SgArgs aq = base(w.wq, qd, d, dec->x, d);
    aq.norm_w = w.attn_norm; aq.y = dec->q; aq.y_stride = qd;
    aq.w2 = static_cast<const uint8_t*>(w.wk); aq.N2 = kvd; aq.y2 = dec->k; aq.y2_stride = kvd;
    aq.w3 = static_cast<const uint8_t*>(w.wv); aq.N3 = kvd; aq.y3 = dec->v; aq.y3_stride = kvd;
    rc = stream_gemv(aq, kind, PRO_RMS, EPI_STORE);
    if (rc) return rc;
    if (!dry) {
        if (rope_on(dec)) {
            rc = b200_rope_forward_cached(dec->q, dec->k, dec->pos, dec->inv_freq, B, dec->H, dec->KV, dec->hd,
                                          dec->rope_type);
            if (rc) return rc;
        }
        kv_append_kernel<<<dim3(ceil_div(kvd, 256), B), 256, 0, st>>>(dec->k, dec->v, w.k_pages, w.v_pages,
                                                                     dec->page_table, dec->pos, dec->max_pages,
                                                                     dec->page, kvd);
        B200_LAUNCH_CHECK("kv_append_kernel");
        rc = b200_attention_decode_paged_fp16(dec->q, w.k_pages, w.v_pages, dec->page_table, dec->len, dec->attn, B,
                                              dec->max_pages, dec->page, dec->H, dec->KV, dec->hd, dec->attn_scale);
        if (rc) return rc;
    }
    SgArgs ao = base(w.wo, d, qd, dec->attn, qd);
    ao.resid = dec->x; ao.y_stride = d; ao.res_mult = dec->res_mult;
    return stream_gemv(ao, kind, PRO_NONE, EPI_RESIDUAL);
}

// Persistent mode: the phase list cut into runs at the attention layers, each run one
// cooperative launch of the persistent kernel; attention mixers and the lm_head on the
// fused few-token kernels between and after them.
static int build_persistent(b200_decoder* dec) {
    B200_REQUIRE(dec->batch == 1, "decoder_configure: the persistent step serves batch 1 (batch is %d)", dec->batch);
    int rc = check_ready(dec);
    if (rc) return rc;
    const int kind = tag_of_qkind(dec->qkind);
    std::vector<PLayer> layers(dec->n_layers);
    std::vector<POp> ops;
    dec->segments.clear();
    int seg_begin = 0;
    ops.push_back({POP_EMBED, 0});
    auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    for (int l = 0; l < dec->n_layers; ++l) {
        const LayerW& w = dec->L[l];
        PLayer& P = layers[l];
        memset(&P, 0, sizeof(P));
        P.attn_norm = w.attn_norm; P.ffn_norm = w.ffn_norm;
        P.mamba_in = static_cast<const uint8_t*>(w.mamba_in); P.mamba_out = static_cast<const uint8_t*>(w.mamba_out);
        P.conv_w = w.conv_w; P.conv_b = w.conv_b; P.dt_bias = w.dt_bias; P.a_log = w.a_log; P.D = w.D;
        P.mamba_norm = w.mamba_norm; P.conv_state = w.conv_state; P.ssm_state = w.ssm_state;
        P.router = w.router; P.router_bias = w.router_bias;
        P.gate = static_cast<const uint8_t*>(w.gate); P.up = static_cast<const uint8_t*>(w.up);
        P.down = static_cast<const uint8_t*>(w.down); P.sh_gate = static_cast<const uint8_t*>(w.sh_gate);
        P.sh_up = static_cast<const uint8_t*>(w.sh_up); P.sh_down = static_cast<const uint8_t*>(w.sh_down);
        P.has_shared = (dec->SH > 0 && w.sh_gate && w.sh_up && w.sh_down) ? 1 : 0;
        B200_REQUIRE(aligned(P.mamba_in) && aligned(P.mamba_out) && aligned(P.router) && aligned(P.gate) && aligned(P.up) &&
                         aligned(P.down) && aligned(P.sh_gate) && aligned(P.sh_up) && aligned(P.sh_down) &&
                         aligned(P.attn_norm) && aligned(P.ffn_norm) && aligned(P.conv_w) && aligned(P.conv_b) &&
                         aligned(P.mamba_norm),
                     "decoder_configure: layer %d: tensors must be 16-byte aligned", l);
        if (dec->types[l] == 0) {
            ops.push_back({POP_MAMBA_A, l});
            ops.push_back({POP_MAMBA_B, l});
        } else {
            dec->segments.push_back({seg_begin, (int)ops.size(), l});
            seg_begin = (int)ops.size();
        }
        ops.push_back({POP_MOE_C, l});
        ops.push_back({POP_MOE_D, l});
        ops.push_back({POP_MOE_E, l});
    }
    dec->segments.push_back({seg_begin, (int)ops.size(), -1});
    PArgs& a = dec->pa;
    a = PArgs();
    a.d = dec->d; a.d_inner = dec->d_inner; a.conv_dim = dec->conv_dim; a.n_heads = dec->mh; a.d_head = dec->mdh;
    a.d_state = dec->mds; a.dconv = dec->mk; a.proj = dec->d_inner + dec->conv_dim + dec->mh;
    a.ne = dec->ne; a.K = dec->K; a.E = dec->E; a.SH = dec->SH; a.vocab = dec->vocab;
    a.eps = dec->eps; a.res_mult = dec->res_mult; a.emb_mult = dec->emb_mult;
    a.n_layers = dec->n_layers;
    for (const b200_decoder::Segment& sg : dec->segments) a.max_ops = std::max(a.max_ops, sg.op_end - sg.op_begin);
    rc = persist_plan(a, kind);
    if (rc) return rc;
    // the attention mixers and the lm_head run on the fused kernels: their tiling must fit too
    for (int l = 0; l < dec->n_layers; ++l)
        if (dec->types[l] != 0) {
            rc = enqueue_attention_fused(dec, dec->L[l], kind, true);
            if (rc) return rc;
        }
    if (!dec->p_layers) {
        rc = dev_alloc(dec, (void**)&dec->p_layers, layers.size() * sizeof(PLayer));
        if (rc) return rc;
        // at most 1 + 5 phases per layer
        rc = dev_alloc(dec, (void**)&dec->p_ops, (size_t)(1 + 5 * dec->n_layers) * sizeof(POp));
        if (rc) return rc;
        char* sync_words = nullptr;
        rc = dev_alloc(dec, (void**)&sync_words, 256);
        if (rc) return rc;
        dec->pa_bar = reinterpret_cast<unsigned long long*>(sync_words);
        dec->pa_done = reinterpret_cast<unsigned int*>(sync_words + 64);
        dec->pa_flag = reinterpret_cast<unsigned int*>(sync_words + 128);
        dec->pa_rt = reinterpret_cast<unsigned int*>(sync_words + 192);
        rc = dev_alloc(dec, (void**)&dec->pa_bcd, (size_t)(2 * dec->mds + dec->mh + 8) * 4);
        if (rc) return rc;
        rc = dev_alloc(dec, (void**)&dec->pa_partials, (size_t)num_sms() * 8);
        if (rc) return rc;
        rc = dev_alloc(dec, (void**)&dec->pa_shout, (size_t)dec->d * 4);
        if (rc) return rc;
    }
    B200_CUDA(cudaMemcpy(dec->p_layers, layers.data(), layers.size() * sizeof(PLayer), cudaMemcpyHostToDevice));
    B200_CUDA(cudaMemcpy(dec->p_ops, ops.data(), ops.size() * sizeof(POp), cudaMemcpyHostToDevice));
    a.layers = dec->p_layers; a.ops = dec->p_ops;
    a.embed = dec->embed; a.len = dec->len; a.pos = dec->pos;
    a.x = dec->x; a.bcd = dec->pa_bcd; a.u = dec->f_u; a.partials = dec->pa_partials; a.logits = dec->f_logits;
    a.sh_act = dec->f_shact; a.sh_out = dec->pa_shout; a.act = dec->f_act;
    a.bar = dec->pa_bar; a.done = dec->pa_done; a.bc_flag = dec->pa_flag; a.rt_flag = dec->pa_rt;
    a.status = stream_status_ptr();
    B200_REQUIRE(a.status, "decoder_configure: status word allocation failed");
    a.spin_limit = dec->test_spin_limit ? dec->test_spin_limit : (1u << 22);
    a.skip_cta = dec->test_skip_cta;
    dec->p_ready = true;
    return B200_OK;
}

static int enqueue_step_persistent(b200_decoder* dec, const int32_t* tokens, int32_t* next) {
    B200_REQUIRE(dec->p_ready, "decoder_step: persistent mode not configured");
    const int kind = tag_of_qkind(dec->qkind);
    cudaStream_t st = stream();
    int rc;
    for (const b200_decoder::Segment& sg : dec->segments) {
        PArgs a = dec->pa;
        a.tok = tokens;
        a.op_begin = sg.op_begin;
        a.op_end = sg.op_end;
        rc = persist_launch(a, kind);
        if (rc) return rc;
        if (sg.attn_layer >= 0) {
            rc = enqueue_attention_fused(dec, dec->L[sg.attn_layer], kind, false);
            if (rc) return rc;
        }
    }
    SgArgs h;
    h.w = reinterpret_cast<const uint8_t*>(dec->lm_head); h.N = dec->vocab; h.K = dec->d; h.M = 1; h.x = dec->x;
    h.x_stride = dec->d; h.eps = dec->eps;
    h.norm_w = dec->final_norm; h.y = dec->logits; h.y_stride = dec->vocab; h.out_scale = 1.0f / dec->logits_scaling;
    rc = stream_gemv(h, KIND_F16, PRO_RMS, EPI_STORE);
    if (rc) return rc;
    return pick_next(dec, dec->logits, tokens, 1, next, 0, 1);
}

static int enqueue(b200_decoder* dec, const int32_t* tokens, int32_t* next) {
    NvtxRange range(dec->fused == 2 ? "b200.step.persistent" : dec->fused ? "b200.step.fused" : "b200.step.per_op");
    if (dec->fused == 2) return enqueue_step_persistent(dec, tokens, next);
    if (dec->fused && dec->batch <= 8) return enqueue_step_fused(dec, tokens, next);
    const int rc = enqueue_step(dec, tokens, next);
    f16_shadow_clear();           // also when a call inside the step failed half-way
    return rc;
}

static int check_ready(const b200_decoder* dec) {
    B200_REQUIRE(dec, "decoder: null handle");
    B200_REQUIRE(dec->embed && dec->lm_head && dec->final_norm, "decoder: embeddings / lm_head / final norm not set");
    B200_REQUIRE(dec->rope_type < 0 || dec->inv_freq, "decoder: RoPE frequency table not set");
    for (int l = 0; l < dec->n_layers; ++l) {
        const LayerW& w = dec->L[l];
        B200_REQUIRE(w.attn_norm && w.ffn_norm && w.router && w.gate && w.up && w.down, "decoder: layer %d: norm or MoE tensors not set", l);
        if (dec->types[l] == 0)
            B200_REQUIRE(w.mamba_in && w.mamba_out && w.conv_w && w.dt_bias && w.a_log && w.D && w.mamba_norm,
                         "decoder: layer %d: Mamba tensors not set", l);
        else
            B200_REQUIRE(w.wq && w.wk && w.wv && w.wo, "decoder: layer %d: attention tensors not set", l);
    }
    return B200_OK;
}

extern "C" {

int b200_decoder_create(b200_decoder** out, int batch, int vocab, int hidden, int n_layers,
                        const int32_t* layer_types_host, int n_heads, int n_kv_heads, int head_dim, int rope_type,
                        int mamba_heads, int mamba_d_head, int mamba_d_state, int mamba_d_conv, int n_experts,
                        int top_k, int expert_dim, int shared_dim, int max_ctx, int kv_page, int qkind,
                        float rms_eps, float embedding_multiplier, float residual_multiplier, float attn_scale,
                        float logits_scaling) {
    B200_REQUIRE(out && layer_types_host, "decoder_create: null pointer");
    B200_REQUIRE(batch > 0 && vocab > 0 && hidden > 0 && n_layers > 0, "decoder_create: bad model dims");
    B200_REQUIRE(qkind >= -1 && qkind <= 3, "decoder_create: unknown qkind %d", qkind);
    B200_REQUIRE(max_ctx > 0 && kv_page > 0, "decoder_create: bad KV geometry");
    B200_REQUIRE(logits_scaling != 0.0f, "decoder_create: logits_scaling must be non-zero");
    b200_decoder* dec = new b200_decoder();
    dec->batch = batch; dec->vocab = vocab; dec->d = hidden; dec->n_layers = n_layers;
    dec->types.assign(layer_types_host, layer_types_host + n_layers);
    dec->H = n_heads; dec->KV = n_kv_heads; dec->hd = head_dim; dec->rope_type = rope_type;
    dec->mh = mamba_heads; dec->mdh = mamba_d_head; dec->mds = mamba_d_state; dec->mk = mamba_d_conv;
    dec->d_inner = mamba_heads * mamba_d_head;
    dec->conv_dim = dec->d_inner + 2 * mamba_d_state;
    dec->ne = n_experts; dec->K = top_k; dec->E = expert_dim; dec->SH = shared_dim;
    dec->page = kv_page;
    dec->max_pages = ceil_div(max_ctx, kv_page);
    dec->max_ctx = dec->max_pages * kv_page;
    dec->qkind = qkind;
    dec->eps = rms_eps; dec->emb_mult = embedding_multiplier; dec->res_mult = residual_multiplier;
    dec->attn_scale = attn_scale > 0.0f ? attn_scale : 1.0f / sqrtf((float)head_dim);
    dec->logits_scaling = logits_scaling;
    dec->L.resize(n_layers);
    *out = dec;
    const int B = batch, d = hidden, qd = n_heads * head_dim, kvd = n_kv_heads * head_dim;
    int rc = 0;
    auto A = [&](void** p, size_t bytes) { if (!rc) rc = dev_alloc(dec, p, bytes); };
    A((void**)&dec->x, (size_t)B * d * 4);
    A((void**)&dec->xb, (size_t)B * d * 4);
    A((void**)&dec->xb16, (size_t)B * d * 2);
    A((void**)&dec->proj, (size_t)B * d * 4);
    A((void**)&dec->q, (size_t)B * std::max(qd, 1) * 4);
    A((void**)&dec->k, (size_t)B * std::max(kvd, 1) * 4);
    A((void**)&dec->v, (size_t)B * std::max(kvd, 1) * 4);
    A((void**)&dec->attn, (size_t)B * std::max(qd, 1) * 4);
    A((void**)&dec->logits, (size_t)B * vocab * 4);
    A((void**)&dec->tok, (size_t)B * 4);
    A((void**)&dec->next, (size_t)B * 4);
    A((void**)&dec->len, (size_t)B * 4);
    A((void**)&dec->pos, (size_t)B * 4);
    A((void**)&dec->page_table, (size_t)B * dec->max_pages * 4);
    {
        MambaDims p{};
        p.n_heads = mamba_heads; p.d_head = mamba_d_head;
        A((void**)&dec->f_gate, (size_t)B * dec->d_inner * 4);
        A((void**)&dec->f_bc, (size_t)B * dec->conv_dim * 4);
        A((void**)&dec->f_dt, (size_t)B * std::max(mamba_heads, 4) * 4);
        A((void**)&dec->f_u, (size_t)B * dec->d_inner * 4);
        dec->f_blocks = std::max(1, mamba_scan_norm_blocks(p));
        A((void**)&dec->f_logits, (size_t)B * std::max(n_experts, 1) * 4);
        A((void**)&dec->f_idx, (size_t)B * std::max(top_k, 1) * 4);
        A((void**)&dec->f_w, (size_t)B * std::max(top_k, 1) * 4);
        A((void**)&dec->f_act, (size_t)B * std::max(top_k * expert_dim, 1) * 4);
        A((void**)&dec->f_shact, (size_t)B * std::max(shared_dim, 1) * 4);
        A((void**)&dec->f_partials, (size_t)B * std::max(1, mamba_scan_norm_blocks(p)) * 8);
    }
    for (int l = 0; l < n_layers && !rc; ++l) {
        LayerW& w = dec->L[l];
        if (dec->types[l] == 0) {
            A((void**)&w.conv_state, (size_t)B * dec->conv_dim * std::max(dec->mk - 1, 1) * 4);
            A((void**)&w.ssm_state, (size_t)B * dec->d_inner * dec->mds * 4);
        } else {
            const size_t bytes = (size_t)B * dec->max_pages * kv_page * kvd * 2;
            A((void**)&w.k_pages, bytes);
            A((void**)&w.v_pages, bytes);
        }
    }
    if (!rc) {
        // sequence b owns pages [b*max_pages, (b+1)*max_pages): identity page table
        std::vector<int32_t> pt((size_t)B * dec->max_pages);
        for (size_t i = 0; i < pt.size(); ++i) pt[i] = (int32_t)i;
        cudaError_t e = cudaMemcpy(dec->page_table, pt.data(), pt.size() * 4, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) rc = cuda_status(e, "decoder_create: page table upload");
    }
    if (!rc) {
        cudaError_t e = cudaMallocHost((void**)&dec->h_tok, (size_t)B * 4);
        // one extra word after the tokens receives the kernels' status word
        if (e == cudaSuccess) e = cudaMallocHost((void**)&dec->h_next, (size_t)(B + 1) * 4);
        if (e != cudaSuccess) rc = cuda_status(e, "decoder_create: pinned staging");
    }
    if (rc) {
        b200_decoder_destroy(dec);
        *out = nullptr;
    }
    return rc;
}

static int seed_sampling(b200_decoder* dec) {
    B200_CUDA(cudaMemsetAsync(dec->hist_total, 0, (size_t)dec->batch * 4, stream()));
    return b200_rng_seed(dec->samp.seed, dec->rng, dec->batch);
}

int b200_decoder_set_sampling(b200_decoder* dec, const b200_sampling* cfg) {
    B200_REQUIRE(dec, "decoder_set_sampling: null handle");
    drop_graph(dec);
    dec->launches = 0;
    if (!cfg) {
        dec->sampling = false;
        return B200_OK;
    }
    b200_sampling c = *cfg;
    b200_sampling_validate(&c);
    if (!dec->hist) {
        int rc = dev_alloc(dec, reinterpret_cast<void**>(&dec->hist), (size_t)dec->batch * DEC_HIST_CAP * 4);
        if (!rc) rc = dev_alloc(dec, reinterpret_cast<void**>(&dec->hist_total), (size_t)dec->batch * 4);
        if (!rc) rc = dev_alloc(dec, reinterpret_cast<void**>(&dec->rng), (size_t)dec->batch * 32);
        if (rc) return rc;
    }
    const size_t need = sample_workspace_bytes(c, dec->vocab, dec->batch);
    if (need > dec->samp_ws_bytes) {
        if (dec->samp_ws) B200_CUDA(cudaFree(dec->samp_ws));
        dec->samp_ws = nullptr;
        dec->samp_ws_bytes = 0;
        B200_CUDA(cudaMalloc(&dec->samp_ws, need));
        dec->samp_ws_bytes = need;
    }
    dec->samp = c;
    dec->sampling = true;
    return seed_sampling(dec);
}

int b200_decoder_score_tokens(b200_decoder* dec, const int32_t* tokens_host, int T, const uint8_t* mask_host,
                              double* mean_nll, int64_t* n_scored) {
    int rc = check_ready(dec);
    if (rc) return rc;
    B200_REQUIRE(tokens_host && mean_nll && T >= 0, "decoder_score_tokens: bad arguments");
    B200_REQUIRE(dec->position == 0, "decoder_score_tokens: the sequences already hold %d tokens (reset first)", dec->position);
    *mean_nll = 0.0;
    if (n_scored) *n_scored = 0;
    if (T < 2) return B200_OK;
    T = std::min(T, std::min(dec->max_ctx, 65535));
    // position i is scored against token i + 1 when that token is supervised; the last
    // position has nothing to predict
    std::vector<int32_t> host((size_t)2 * T);
    for (int i = 0; i < T; ++i) {
        host[i] = tokens_host[i];
        const bool supervised = i + 1 < T && (!mask_host || mask_host[i + 1] != 0);
        host[T + i] = supervised ? tokens_host[i + 1] : -100;
        B200_REQUIRE(host[T + i] < dec->vocab, "decoder_score_tokens: token %d at %d is outside the vocabulary", host[T + i], i + 1);
    }
    // ids, targets and the accumulator in a buffer of their own (the library's workspaces are
    // all in use by the prompt kernels)
    const size_t acc_off = ((size_t)2 * T * 4 + 255) & ~(size_t)255;
    void* buf = nullptr;
    B200_CUDA(cudaMalloc(&buf, acc_off + 256));
    int32_t* ids = static_cast<int32_t*>(buf);
    double* acc = reinterpret_cast<double*>(static_cast<char*>(buf) + acc_off);
    unsigned long long out[2] = {0, 0};
    auto run = [&]() -> int {
        B200_CUDA(cudaMemcpyAsync(ids, host.data(), (size_t)2 * T * 4, cudaMemcpyHostToDevice, stream()));
        B200_CUDA(cudaMemsetAsync(acc, 0, 32, stream()));
        const int prc = prefill(dec, ids, T, nullptr, 0, 1, ids + T, acc);
        if (prc) return prc;
        B200_CUDA(cudaMemcpyAsync(out, acc, 16, cudaMemcpyDeviceToHost, stream()));
        B200_CUDA(cudaStreamSynchronize(stream()));
        return B200_OK;
    };
    rc = run();
    cudaFree(buf);
    if (rc) return rc;
    if (dec->graph && dec->ws_generation != workspace_generation()) {
        drop_graph(dec);
        dec->launches = 0;
    }
    dec->position = T;
    double sum;
    memcpy(&sum, &out[0], 8);
    const int64_t n = (int64_t)out[1];
    if (n_scored) *n_scored = n;
    *mean_nll = n > 0 ? sum / (double)n : 0.0;
    return B200_OK;
}

int b200_decoder_destroy(b200_decoder* dec) {
    if (!dec) return B200_OK;
    drop_graph(dec);
    if (dec->own_stream) cudaStreamDestroy(dec->own_stream);
    for (void* p : dec->owned) cudaFree(p);
    if (dec->samp_ws) cudaFree(dec->samp_ws);
    if (dec->h_tok) cudaFreeHost(dec->h_tok);
    if (dec->h_next) cudaFreeHost(dec->h_next);
    delete dec;
    return B200_OK;
}

int b200_decoder_set_tensor(b200_decoder* dec, int layer, int id, const void* p) {
    B200_REQUIRE(dec, "decoder_set_tensor: null handle");
    drop_graph(dec);
    if (dec->fused == 2) dec->fused = 0;        // the layer table on the device is stale: configure again
    dec->p_ready = false;
    if (layer < 0) {
        switch (id) {
            case B200_T_EMBED: dec->embed = static_cast<const uint16_t*>(p); return B200_OK;
            case B200_T_FINAL_NORM: dec->final_norm = static_cast<const float*>(p); return B200_OK;
            case B200_T_LM_HEAD: dec->lm_head = static_cast<const uint16_t*>(p); return B200_OK;
            case B200_T_ROPE_INV_FREQ: dec->inv_freq = static_cast<const float*>(p); return B200_OK;
            default: return fail(B200_EINVAL, "decoder_set_tensor: %d is not a model-level tensor", id);
        }
    }
    B200_REQUIRE(layer < dec->n_layers, "decoder_set_tensor: layer %d out of range", layer);
    LayerW& w = dec->L[layer];
    const float* f = static_cast<const float*>(p);
    switch (id) {
        case B200_T_ATTN_NORM: w.attn_norm = f; break;
        case B200_T_FFN_NORM: w.ffn_norm = f; break;
        case B200_T_MAMBA_IN: w.mamba_in = p; break;
        case B200_T_MAMBA_CONV_W: w.conv_w = f; break;
        case B200_T_MAMBA_CONV_B: w.conv_b = f; break;
        case B200_T_MAMBA_DT_BIAS: w.dt_bias = f; break;
        case B200_T_MAMBA_A_LOG: w.a_log = f; break;
        case B200_T_MAMBA_D: w.D = f; break;
        case B200_T_MAMBA_NORM: w.mamba_norm = f; break;
        case B200_T_MAMBA_OUT: w.mamba_out = p; break;
        case B200_T_WQ: w.wq = p; break;
        case B200_T_WK: w.wk = p; break;
        case B200_T_WV: w.wv = p; break;
        case B200_T_WO: w.wo = p; break;
        case B200_T_ROUTER: w.router = f; break;
        case B200_T_ROUTER_BIAS: w.router_bias = f; break;
        case B200_T_MOE_GATE: w.gate = p; break;
        case B200_T_MOE_UP: w.up = p; break;
        case B200_T_MOE_DOWN: w.down = p; break;
        case B200_T_SH_GATE: w.sh_gate = p; break;
        case B200_T_SH_UP: w.sh_up = p; break;
        case B200_T_SH_DOWN: w.sh_down = p; break;
        default: return fail(B200_EINVAL, "decoder_set_tensor: unknown tensor id %d", id);
    }
    return B200_OK;
}

int b200_decoder_reset(b200_decoder* dec) {
    B200_REQUIRE(dec, "decoder_reset: null handle");
    cudaStream_t st = stream();
    const int B = dec->batch;
    B200_CUDA(cudaMemsetAsync(dec->len, 0, (size_t)B * 4, st));
    for (int l = 0; l < dec->n_layers; ++l) {
        LayerW& w = dec->L[l];
        if (dec->types[l] == 0) {
            B200_CUDA(cudaMemsetAsync(w.conv_state, 0, (size_t)B * dec->conv_dim * std::max(dec->mk - 1, 1) * 4, st));
            B200_CUDA(cudaMemsetAsync(w.ssm_state, 0, (size_t)B * dec->d_inner * dec->mds * 4, st));
        }
    }
    dec->position = 0;
    if (dec->sampling) return seed_sampling(dec);
    return B200_OK;
}

int b200_decoder_configure(b200_decoder* dec, int fused, int use_graph) {
    B200_REQUIRE(dec, "decoder_configure: null handle");
    B200_REQUIRE(fused >= 0 && fused <= 2, "decoder_configure: fused must be 0, 1 or 2");
    drop_graph(dec);
    if (fused == 2) {
        const int rc = build_persistent(dec);
        if (rc) return rc;
    } else if (fused && dec->batch <= 8) {
        // every matrix of the model must fit the streaming kernels' tiling: say so now,
        // not in the middle of a step
        const int rc = enqueue_step_fused(dec, nullptr, nullptr, true);
        if (rc) return rc;
    }
    dec->fused = fused;
    dec->use_graph = use_graph ? 1 : 0;
    dec->launches = 0;
    return B200_OK;
}

int b200_decoder_step(b200_decoder* dec, const int32_t* tokens_dev, int32_t* next_dev) {
    int rc = check_ready(dec);
    if (rc) return rc;
    B200_REQUIRE(tokens_dev && next_dev, "decoder_step: null pointer");
    B200_REQUIRE(dec->position < dec->max_ctx, "decoder_step: context full (%d tokens)", dec->max_ctx);
    if (!dec->use_graph) {
        const unsigned long long before = g_kernel_launches;
        rc = enqueue(dec, tokens_dev, next_dev);
        dec->launches = (int)(g_kernel_launches - before);
        if (rc) return rc;
        dec->position += 1;
        return B200_OK;
    }
    // A captured step holds the addresses of the library's workspaces: once one of them
    // has been reallocated or released the recording is stale.
    if (dec->graph && dec->ws_generation != workspace_generation()) {
        drop_graph(dec);
        dec->launches = 0;          // one eager step first: it sizes the workspaces again
    }
    if (!dec->graph || dec->graph_tok != tokens_dev || dec->graph_next != next_dev) {
        drop_graph(dec);
        // Workspaces grow with cudaMalloc, which cannot run inside a capture.  The
        // first step of a configuration therefore runs eagerly (sizing every
        // workspace); the capture happens on the second.
        if (dec->launches == 0) {
            const unsigned long long before = g_kernel_launches;
            rc = enqueue(dec, tokens_dev, next_dev);
            dec->launches = (int)(g_kernel_launches - before);
            if (rc) return rc;
            dec->position += 1;
            return B200_OK;
        }
        if (!dec->own_stream) B200_CUDA(cudaStreamCreateWithFlags(&dec->own_stream, cudaStreamNonBlocking));
        cudaStream_t prev = stream();
        b200_set_stream(dec->own_stream);
        cudaGraph_t g = nullptr;
        cudaError_t e = cudaStreamBeginCapture(dec->own_stream, cudaStreamCaptureModeThreadLocal);
        if (e == cudaSuccess) {
            const unsigned long long before = g_kernel_launches;
            rc = enqueue(dec, tokens_dev, next_dev);
            dec->launches = (int)(g_kernel_launches - before);
            e = cudaStreamEndCapture(dec->own_stream, &g);
        }
        b200_set_stream(prev);
        if (rc) { if (g) cudaGraphDestroy(g); return rc; }
        if (e != cudaSuccess) return cuda_status(e, "decoder_step: stream capture");
        e = cudaGraphInstantiate(&dec->graph, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) return cuda_status(e, "decoder_step: cudaGraphInstantiate");
        dec->graph_tok = tokens_dev;
        dec->graph_next = next_dev;
        dec->ws_generation = workspace_generation();
    }
    B200_CUDA(cudaGraphLaunch(dec->graph, stream()));
    dec->position += 1;
    return B200_OK;
}

int b200_decoder_step_host(b200_decoder* dec, const int32_t* tokens_host, int32_t* next_host) {
    B200_REQUIRE(dec && tokens_host && next_host, "decoder_step_host: null pointer");
    const size_t bytes = (size_t)dec->batch * 4;
    memcpy(dec->h_tok, tokens_host, bytes);
    B200_CUDA(cudaMemcpyAsync(dec->tok, dec->h_tok, bytes, cudaMemcpyHostToDevice, stream()));
    int rc = b200_decoder_step(dec, dec->tok, dec->next);
    if (rc) return rc;
    B200_CUDA(cudaMemcpyAsync(dec->h_next, dec->next, bytes, cudaMemcpyDeviceToHost, stream()));
    int* status_dev = stream_status_ptr();
    dec->h_next[dec->batch] = 0;
    if (status_dev)
        B200_CUDA(cudaMemcpyAsync(dec->h_next + dec->batch, status_dev, 4, cudaMemcpyDeviceToHost, stream()));
    B200_CUDA(cudaStreamSynchronize(stream()));
    memcpy(next_host, dec->h_next, bytes);
    if (dec->h_next[dec->batch] != 0) return stream_status_check("decoder_step_host");
    return B200_OK;
}

int b200_decoder_prefill(b200_decoder* dec, const int32_t* tokens_dev, int T, int32_t* next_dev) {
    int rc = check_ready(dec);
    if (rc) return rc;
    B200_REQUIRE(tokens_dev && T >= 1, "decoder_prefill: bad arguments");
    B200_REQUIRE(dec->position == 0, "decoder_prefill: the sequences already hold %d tokens (reset first)", dec->position);
    B200_REQUIRE(T <= dec->max_ctx, "decoder_prefill: %d tokens exceed the context of %d", T, dec->max_ctx);
    B200_REQUIRE((int64_t)dec->batch * T <= 0x7fffffff / std::max(dec->K, 1), "decoder_prefill: batch * T too large");
    B200_REQUIRE(dec->batch <= 65535 && T <= 65535, "decoder_prefill: batch and T must be <= 65535");
    // Groups of sequences of at most PREFILL_GROUP_TOKENS tokens: bounds the prompt path's
    // workspaces (tens of bytes per token and layer width) whatever the batch is.
    const int group = std::max(1, std::min(dec->batch, PREFILL_GROUP_TOKENS / T));
    for (int b0 = 0; b0 < dec->batch; b0 += group) {
        const int B = std::min(group, dec->batch - b0);
        rc = prefill(dec, tokens_dev + (int64_t)b0 * T, T, next_dev ? next_dev + b0 : nullptr, b0, B);
        if (rc) return rc;
    }
    if (dec->graph && dec->ws_generation != workspace_generation()) {
        drop_graph(dec);
        dec->launches = 0;
    }
    dec->position = T;
    return B200_OK;
}

int b200_decoder_prefill_ragged(b200_decoder* dec, const int32_t* tokens_dev, const int32_t* lengths_host,
                                int32_t* next_dev) {
    int rc = check_ready(dec);
    if (rc) return rc;
    B200_REQUIRE(tokens_dev && lengths_host, "decoder_prefill_ragged: null pointer");
    B200_REQUIRE(dec->position == 0, "decoder_prefill_ragged: the sequences already hold %d tokens (reset first)", dec->position);
    int longest = 0;
    for (int b = 0; b < dec->batch; ++b) {
        B200_REQUIRE(lengths_host[b] >= 1 && lengths_host[b] <= dec->max_ctx,
                     "decoder_prefill_ragged: sequence %d has %d tokens (1 .. %d allowed)", b, lengths_host[b], dec->max_ctx);
        longest = std::max(longest, lengths_host[b]);
    }
    // Groups of consecutive sequences of at most PREFILL_GROUP_TOKENS tokens together (a longer
    // sequence forms a group of its own): bounds the prompt path's workspaces.
    std::vector<int32_t> h;            // host image of one group's tables
    int32_t* tables = nullptr;         // its device copy, sized for the largest group
    size_t tables_cap = 0;
    int64_t tok0 = 0;
    for (int b0 = 0; b0 < dec->batch && rc == B200_OK;) {
        int B = 0;
        int64_t rows = 0;
        while (b0 + B < dec->batch && (B == 0 || rows + lengths_host[b0 + B] <= PREFILL_GROUP_TOKENS)) rows += lengths_host[b0 + B++];
        int n_chunks = 0;
        for (int b = 0; b < B; ++b) n_chunks += ceil_div(lengths_host[b0 + b], SSD_Q);
        // layout of the tables (int32 words): seq_off [B+1] | seq_chunk0 [B+1] | pos [rows] | seq [rows] | chunks [2 n_chunks]
        const size_t o_off = 0, o_c0 = o_off + B + 1, o_pos = (o_c0 + B + 1 + 3) & ~(size_t)3, o_seq = o_pos + rows,
                     o_chunks = (o_seq + rows + 3) & ~(size_t)3, words = o_chunks + 2 * (size_t)n_chunks;
        h.assign(words, 0);
        int64_t r = 0;
        int c = 0;
        for (int b = 0; b < B; ++b) {
            const int n = lengths_host[b0 + b];
            h[o_off + b] = (int32_t)r;
            h[o_c0 + b] = c;
            for (int t = 0; t < n; ++t) {
                h[o_pos + r + t] = t;
                h[o_seq + r + t] = b;
            }
            for (int t = 0; t < n; t += SSD_Q, ++c) {
                h[o_chunks + 2 * c] = (int32_t)(r + t);
                h[o_chunks + 2 * c + 1] = std::min(SSD_Q, n - t);
            }
            r += n;
        }
        h[o_off + B] = (int32_t)r;
        h[o_c0 + B] = c;
        if (words > tables_cap) {
            if (tables) cudaFree(tables);
            tables = nullptr;
            cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&tables), words * 4);
            if (e != cudaSuccess) return cuda_status(e, "decoder_prefill_ragged: cudaMalloc");
            tables_cap = words;
        }
        cudaError_t e = cudaMemcpyAsync(tables, h.data(), words * 4, cudaMemcpyHostToDevice, stream());
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream());      // h is reused by the next group
        if (e != cudaSuccess) { rc = cuda_status(e, "decoder_prefill_ragged: table upload"); break; }
        SeqLayout lay;
        lay.n_seq = B;
        lay.rows = rows;
        lay.n_chunks = n_chunks;
        lay.seq_off = tables + o_off;
        lay.seq_chunk0 = tables + o_c0;
        lay.pos = tables + o_pos;
        lay.seq = tables + o_seq;
        lay.chunks = reinterpret_cast<const int2*>(tables + o_chunks);
        lay.host_off = h.data() + o_off;
        rc = prefill(dec, tokens_dev + tok0, 0, next_dev ? next_dev + b0 : nullptr, b0, B, nullptr, nullptr, &lay);
        tok0 += rows;
        b0 += B;
    }
    if (tables) {
        cudaStreamSynchronize(stream());       // the kernels of the last group still read the tables
        cudaFree(tables);
    }
    if (rc) return rc;
    if (dec->graph && dec->ws_generation != workspace_generation()) {
        drop_graph(dec);
        dec->launches = 0;
    }
    dec->position = longest;
    return B200_OK;
}

int b200_decoder_set_rope_refresh(b200_decoder* dec, int as_reference) {
    B200_REQUIRE(dec, "decoder_set_rope_refresh: null handle");
    drop_graph(dec);
    dec->rope_refresh_as_reference = as_reference ? 1 : 0;
    return B200_OK;
}

int b200_decoder_test_barrier(b200_decoder* dec, int spin_limit, int skip_cta) {
    B200_REQUIRE(dec && spin_limit >= 0, "decoder_test_barrier: bad arguments");
    drop_graph(dec);
    dec->test_spin_limit = (unsigned)spin_limit;
    dec->test_skip_cta = skip_cta;
    dec->pa.spin_limit = spin_limit ? (unsigned)spin_limit : (1u << 22);
    dec->pa.skip_cta = skip_cta;
    return B200_OK;
}

int b200_decoder_phase_trace(b200_decoder* dec, int cta, uint64_t* stamps_host, int cap, int* n_phases) {
    B200_REQUIRE(dec && dec->p_ready, "decoder_phase_trace: the persistent mode is not configured");
    const int n_ops = dec->segments.empty() ? 0 : dec->segments.back().op_end;
    if (n_phases) *n_phases = n_ops;
    if (!stamps_host) {
        // arm (cta >= 0) or disarm (cta < 0) the timers
        drop_graph(dec);
        if (cta >= 0 && !dec->pa_trace) {
            int rc = dev_alloc(dec, (void**)&dec->pa_trace, (size_t)n_ops * PS_TRACE_SLOTS * 8);
            if (rc) return rc;
        }
        dec->pa.trace = cta >= 0 ? dec->pa_trace : nullptr;
        dec->pa.trace_cta = cta >= 0 ? cta : 0;
        return B200_OK;
    }
    B200_REQUIRE(dec->pa_trace && cap >= n_ops * PS_TRACE_SLOTS, "decoder_phase_trace: timers not armed or buffer too small");
    B200_CUDA(cudaStreamSynchronize(stream()));
    B200_CUDA(cudaMemcpy(stamps_host, dec->pa_trace, (size_t)n_ops * PS_TRACE_SLOTS * 8, cudaMemcpyDeviceToHost));
    return B200_OK;
}

int b200_decoder_logits(b200_decoder* dec, const float** logits_dev) {
    B200_REQUIRE(dec && logits_dev, "decoder_logits: null pointer");
    *logits_dev = dec->logits;
    return B200_OK;
}
int b200_decoder_position(b200_decoder* dec, int* position) {
    B200_REQUIRE(dec && position, "decoder_position: null pointer");
    *position = dec->position;
    return B200_OK;
}
int b200_decoder_launches_per_step(b200_decoder* dec, int* launches) {
    B200_REQUIRE(dec && launches, "decoder_launches_per_step: null pointer");
    *launches = dec->launches;
    return B200_OK;
}

static double packed_bytes(int qkind, double rows, double cols) {
    if (qkind < 0) return rows * cols * 2.0;
    const double be = qkind == 3 ? 256.0 : 32.0;
    const double bb = qkind == 0 ? 18.0 : qkind == 1 ? 20.0 : qkind == 2 ? 34.0 : 144.0;
    return rows * cols / be * bb;
}

int b200_decoder_step_bytes(b200_decoder* dec, double* bytes) {
    B200_REQUIRE(dec && bytes, "decoder_step_bytes: null pointer");
    const double B = dec->batch, d = dec->d;
    const int q = dec->qkind;
    double total = d * 2.0 * B;                              // embedding rows
    total += (double)dec->vocab * d * 2.0;                   // lm_head
    total += d * 4.0;                                        // final norm
    const double tokens_in_cache = dec->position + 1;
    // experts touched by a step: at most all of them, at most batch*K
    const double routed = std::min((double)dec->ne, B * dec->K);
    for (int l = 0; l < dec->n_layers; ++l) {
        total += 2.0 * d * 4.0;                              // two norms
        if (dec->types[l] == 0) {
            const double proj = dec->d_inner + dec->conv_dim + dec->mh;
            total += packed_bytes(q, proj, d) + packed_bytes(q, d, dec->d_inner);
            total += (double)dec->conv_dim * (dec->mk + 1) * 4.0 + dec->mh * 12.0 + dec->d_inner * 4.0;
            total += B * 2.0 * ((double)dec->d_inner * dec->mds * 4.0 + (double)dec->conv_dim * (dec->mk - 1) * 4.0);
        } else {
            const double qd = (double)dec->H * dec->hd, kvd = (double)dec->KV * dec->hd;
            total += packed_bytes(q, qd + 2 * kvd, d) + packed_bytes(q, d, qd);
            total += B * tokens_in_cache * 2.0 * kvd * 2.0;  // K and V rows, fp16
        }
        total += (double)dec->ne * d * 4.0 + dec->ne * 4.0;  // router + bias
        total += routed * 3.0 * packed_bytes(q, dec->E, d);
        if (dec->SH > 0) total += 3.0 * packed_bytes(q, dec->SH, d);
    }
    *bytes = total;
    return B200_OK;
}

}  // extern "C"
