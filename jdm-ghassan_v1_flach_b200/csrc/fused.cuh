// Host interface of the fused decode-step kernels (fused_gemv.cu, fused_moe.cu).
#pragma once

#include "stream.cuh"

namespace b200 {

struct MambaDims {
    int d, d_inner, conv_dim, n_heads, d_head, d_state, k, proj;
    float eps;
};

// Sequences of different lengths packed back to back (row = token): what the sequence-aware
// prompt kernels need to know.  Device arrays unless noted.
constexpr int SSD_Q = 128;                // steps per chunk of the chunked Mamba-2 scan
struct SeqLayout {
    int n_seq = 0;
    int64_t rows = 0;                     // tokens of all sequences
    int n_chunks = 0;
    const int32_t* seq_off = nullptr;     // [n_seq + 1] first row of each sequence
    const int32_t* pos = nullptr;         // [rows] position of a row inside its sequence
    const int32_t* seq = nullptr;         // [rows] sequence a row belongs to
    const int2* chunks = nullptr;         // [n_chunks] (first row, steps <= SSD_Q); no chunk crosses a sequence boundary
    const int32_t* seq_chunk0 = nullptr;  // [n_seq + 1] first chunk of each sequence
    const int32_t* host_off = nullptr;    // host copy of seq_off
};

enum { PRO_NONE = 0, PRO_RMS = 1 };
enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_INPROJ = 2 };

// One streamed matrix-vector product y[M,N] = f(x)[M,K] . W^T for M <= 8 tokens.
struct SgArgs {
    const uint8_t* w = nullptr;     // [N,K] in the kernel's weight kind
    int N = 0, K = 0, M = 0;
    const float* x = nullptr;       // [M, x_stride]
    int x_stride = 0;
    const float* norm_w = nullptr;  // PRO_RMS: x <- x * inv_rms(x) * norm_w
    float eps = 0.0f;
    // optional per-token scalar on the dot products: 1/sqrt(sum(partials)/in_dim + eps)
    const double* in_partials = nullptr;
    int n_partials = 0, in_dim = 1;
    float out_scale = 1.0f;         // EPI_STORE: y = acc * out_scale
    float* y = nullptr;             // EPI_STORE output, rows y_stride apart
    int y_stride = 0;
    // EPI_STORE only: up to two more matrices over the same activations in the same launch
    // (the q / k / v projections of an attention layer): [N2,K] -> y2, [N3,K] -> y3, same
    // kind, same y_stride convention (rows y2_stride / y3_stride apart)
    const uint8_t *w2 = nullptr, *w3 = nullptr;
    int N2 = 0, N3 = 0;
    float *y2 = nullptr, *y3 = nullptr;
    int y2_stride = 0, y3_stride = 0;
    int t1 = 0, t2 = 0;             // first tile of the second / third matrix (filled by stream_gemv())
    float* resid = nullptr;         // EPI_RESIDUAL: resid += res_mult * acc (rows y_stride apart)
    float res_mult = 1.0f;
    // EPI_INPROJ (Mamba in_proj): gate | conv step | dt
    MambaDims p = {};
    const float *conv_w = nullptr, *conv_b = nullptr;
    float *conv_state = nullptr, *gate = nullptr, *bc = nullptr, *dt_raw = nullptr;
    // filled by stream_gemv()
    int rows_per_tile = 0, num_tiles = 0, stage_bytes = 0, n_stages = 0;
    int64_t row_bytes = 0;
    int* status = nullptr;
    bool dry = false;               // validate shapes and tiling, launch nothing
};

int stream_gemv(SgArgs a, int kind, int pro, int epi);

// Whole-sequence Mamba-2 layer (mamba.cu).  kind: template tag of the projections'
// storage.  conv_state_out (optional) [B, conv_dim, k-1] receives the convolution
// window a following decode step continues from.  x16 (optional): the same activations
// already rounded to fp16 rows [B*T, d] by their producer, used instead of converting x
// when the projection runs as a tensor-core GEMM.  lay (optional): the B sequences have
// different lengths and lie packed as lay describes (T is ignored); state and
// conv_state_out stay [B, ...].
int mamba2_forward(const float* x, const void* w_in, const float* conv_w, const float* conv_b, const float* dt_bias,
                   const float* a_log, const float* D, const float* norm_w, const void* w_out, float* state, float* out,
                   int B, int T, MambaDims p, int kind, float* conv_state_out = nullptr, const void* x16 = nullptr,
                   const SeqLayout* lay = nullptr);

// Decode state update; partials: [batch, mamba_scan_norm_blocks()] doubles.
int mamba_scan_norm(const float* bc, const float* dt_raw, const float* gate, const float* dt_bias,
                    const float* a_log, const float* D, const float* norm_w, float* ssm_state, float* u_out,
                    double* partials, int batch, const MambaDims& p);
int mamba_scan_norm_blocks(const MambaDims& p);

// MoE layer on M <= 8 tokens: resid += res_mult * moe(rmsnorm(x) * norm_w).
struct MoeFusedArgs {
    const float* x = nullptr;        // [M, d] pre-norm residual stream
    const float* norm_w = nullptr;
    float eps = 0.0f;
    const float *router_w = nullptr, *router_bias = nullptr;
    const uint8_t *gates = nullptr, *ups = nullptr, *downs = nullptr, *sh_g = nullptr, *sh_u = nullptr, *sh_d = nullptr;
    float* logits = nullptr;         // [M, ne] scratch
    int32_t* idx = nullptr;          // [M, K]
    float* w = nullptr;              // [M, K]
    float* probs_out = nullptr;      // optional [M, ne]
    float* act = nullptr;            // [M, K, E] scratch
    float* sh_act = nullptr;         // [M, SH] scratch
    float* resid = nullptr;          // [M, d], updated in place
    float res_mult = 1.0f;
    int M = 0, d = 0, E = 0, ne = 0, K = 0, SH = 0;
    // filled per phase
    int rows_per_tile = 0, stage_bytes = 0, n_stages = 0;
    int* status = nullptr;
    int* route_counter = nullptr;   // router tiles finished so far in this layer (returns to 0)
    bool dry = false;               // validate shapes and tiling, launch nothing
};
int moe_fused(MoeFusedArgs a, int kind);

}  // namespace b200
