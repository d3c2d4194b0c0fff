// Host interface of the persistent decode-step kernel (step_persistent.cu): one
// cooperative launch walks a list of layer phases for a single token with all CTAs
// resident, a weight stream that runs on across phase boundaries and bounded grid
// barriers between the phases.
#pragma once

#include "fused.cuh"

namespace b200 {

// Device-resident description of one layer (pointers into the caller's weights and the
// decoder's state).  Attention projections are not listed: attention layers run through
// the per-phase kernels between two persistent segments.
struct PLayer {
    const float *attn_norm, *ffn_norm;
    const uint8_t *mamba_in, *mamba_out;
    const float *conv_w, *conv_b, *dt_bias, *a_log, *D, *mamba_norm;
    float *conv_state, *ssm_state;
    const float *router, *router_bias;
    const uint8_t *gate, *up, *down, *sh_gate, *sh_up, *sh_down;
    int has_shared;
    int pad_;
};

// Phases.  Every phase but the last of a launch ends with a grid barrier.
enum {
    POP_EMBED = 0,    // x = embed[token] * multiplier; position bookkeeping
    POP_MAMBA_A = 1,  // RMSNorm -> in_proj -> conv step -> state update -> gated-norm statistics
    POP_MAMBA_B = 2,  // out_proj (scaled by the gated-norm statistic) -> residual
    POP_MOE_C = 3,    // RMSNorm -> router logits (exact fp32 order) || shared gate/up (SwiGLU)
    POP_MOE_D = 4,    // routing (softmax, top-K) -> shared down || routed gate/up (SwiGLU)
    POP_MOE_E = 5,    // routed down, weighted combine with the shared expert, residual
};
struct POp {
    int op, layer;
};

constexpr int PS_MAX_STAGES = 8;
constexpr int PS_TRACE_SLOTS = 8;           // phase start, activations staged, tiles done, barrier passed
constexpr int PS_SMEM_MAX = 224 * 1024;     // dynamic shared memory of the one CTA per SM

struct PArgs {
    const PLayer* layers = nullptr;
    const POp* ops = nullptr;
    int op_begin = 0, op_end = 0;
    int n_layers = 0, max_ops = 0;       // layers in the table; most phases any launch will carry
    // model
    int d = 0, d_inner = 0, conv_dim = 0, n_heads = 0, d_head = 0, d_state = 0, dconv = 0, proj = 0;
    int ne = 0, K = 0, E = 0, SH = 0, vocab = 0;
    float eps = 0.f, res_mult = 1.f, emb_mult = 1.f;
    // token in / embedding
    const int32_t* tok = nullptr;
    const uint16_t* embed = nullptr;
    int32_t *len = nullptr, *pos = nullptr;
    // activations exchanged between phases (global memory, L2 resident)
    float* x = nullptr;            // [d] residual stream
    float* bcd = nullptr;          // [2 * d_state + n_heads] conv'd B, C and raw dt
    float* u = nullptr;            // [d_inner] y * silu(gate) * norm_w
    double* partials = nullptr;    // [grid] sum of squares of y * silu(gate) per CTA
    float* logits = nullptr;       // [ne]
    float* sh_act = nullptr;       // [SH]
    float* sh_out = nullptr;       // [d]
    float* act = nullptr;          // [K, E]
    // synchronisation words (zero between launches)
    unsigned long long* bar = nullptr;   // grid-barrier arrivals
    unsigned int* done = nullptr;        // CTAs that left the kernel
    unsigned int* bc_flag = nullptr;     // B/C/dt tiles finished
    unsigned int* rt_flag = nullptr;     // router logits published (one count per expert and layer)
    int* status = nullptr;               // 0 = ok, 1 = a bounded wait ran out
    unsigned int spin_limit = 1u << 22;  // iterations of a global-memory wait
    int skip_cta = -1;                   // test hook: this CTA leaves at its first barrier without arriving
    // optional phase timers: [n_ops][PS_TRACE_SLOTS] globaltimer stamps written by CTA trace_cta
    unsigned long long* trace = nullptr;
    int trace_cta = 0;
    // shared-memory plan (bytes from the start of dynamic shared memory)
    int stage_bytes = 0, n_stages = 0;
    int off_xa1 = 0, off_xa2 = 0, off_xa3 = 0, off_nw = 0, off_gs = 0, off_red = 0, off_route = 0, off_bcd = 0,
        off_prog = 0, off_ctl = 0, smem_bytes = 0;
};

// Fills the shared-memory plan for `kind` (template tag) and checks that every phase's
// tiles fit; B200_EUNSUPPORTED with a message otherwise.
int persist_plan(PArgs& a, int kind);
// Launches ops [a.op_begin, a.op_end) on the library's current stream.
int persist_launch(const PArgs& a, int kind);

}  // namespace b200
