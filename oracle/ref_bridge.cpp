// extern "C" bridge over the reference engine's own CPU objects.
//
// TEST INFRASTRUCTURE ONLY.  oracle/Makefile compiles the reference's CPU sources
// where they lie (nothing is copied) together with this file into
// oracle/_ref/libgai_ref.so.  The bridge lets the Python tests and the benchmark's
// reference arm call gai::cpu::*, gai::ops::*(Device::CPU) and gai::quant::*
// directly, so the oracle restatement can be pinned against the real thing and the
// golden fixtures can be generated from it.  The product never loads it.
#include "core/ops.h"
#include "core/ops_cpu.h"
#include "core/tensor.h"
#include "quantization/quantize.h"

#include <cstring>
#include <string>

#ifdef GAI_OPENMP
#include <omp.h>
#endif

using namespace gai;

#define REF_API extern "C" __attribute__((visibility("default")))

static thread_local std::string g_err;

template <typename F>
static int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

REF_API const char* ref_last_error() { return g_err.c_str(); }

REF_API int ref_num_threads() {
#ifdef GAI_OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// kind: 0 Q4_0, 1 Q4_1, 2 Q8_0
REF_API int ref_quantize(const float* src, void* dst, i64 n, int kind) {
    return guarded([&] {
        if (kind == 0) quant::quantize_q4_0(src, dst, n);
        else if (kind == 1) quant::quantize_q4_1(src, dst, n);
        else quant::quantize_q8_0(src, dst, n);
    });
}

REF_API int ref_dequantize_f32(const void* src, float* dst, i64 n, int kind) {
    return guarded([&] {
        if (kind == 0) quant::dequantize_q4_0(src, dst, n);
        else if (kind == 1) quant::dequantize_q4_1(src, dst, n);
        else quant::dequantize_q8_0(src, dst, n);
    });
}

// ops::quant_materialize on the CPU device: packed -> fp16
REF_API int ref_quant_materialize(const void* packed, u16* dst, i64 n, int kind) {
    return guarded([&] {
        const u16* p = ops::quant_materialize(Device::CPU, packed, kind, n, 0);
        std::memcpy(dst, p, sizeof(u16) * static_cast<size_t>(n));
    });
}

REF_API int ref_linear_q4(const float* x, const void* w, float* y, int M, int K, int N, int kind) {
    return guarded([&] { ops::linear_forward_q4(Device::CPU, x, w, y, M, K, N, kind); });
}

REF_API int ref_linear_f32(const float* x, const float* w, float* y, int M, int K, int N) {
    return guarded([&] { cpu::linear_forward(x, w, y, M, K, N); });
}

REF_API int ref_linear_f16(const float* x, const u16* w, float* y, int M, int K, int N) {
    return guarded([&] { cpu::linear_forward_fp16(x, w, y, M, K, N); });
}

REF_API int ref_embedding(const i32* ids, const void* table, int half, float* out, i64 ntok,
                          int dim, int vocab) {
    return guarded([&] {
        if (half) cpu::embedding_forward_half(ids, static_cast<const u16*>(table), out, ntok, dim, vocab);
        else cpu::embedding_forward(ids, static_cast<const float*>(table), out, ntok, dim, vocab);
    });
}

REF_API int ref_rmsnorm(const float* x, const float* w, float* out, float* rrms, i64 rows, int dim,
                        float eps) {
    return guarded([&] { cpu::rmsnorm_forward(x, w, out, rrms, rows, dim, eps); });
}

REF_API int ref_rope_cached(float* q, float* k, const i32* pos, const float* inv_freq, i64 ntok,
                            int n_heads, int n_kv, int head_dim, int rope_type) {
    return guarded([&] {
        cpu::rope_forward_cached(q, k, pos, inv_freq, ntok, n_heads, n_kv, head_dim, rope_type);
    });
}

REF_API int ref_swiglu(const float* g, const float* u, float* out, i64 n) {
    return guarded([&] { cpu::swiglu_forward(g, u, out, n); });
}

REF_API int ref_argmax(const float* logits, int V, i32* out) {
    return guarded([&] { *out = cpu::argmax_token(logits, V); });
}

REF_API int ref_topk(const float* logits, int V, int K, float* vals, i32* ids) {
    return guarded([&] { cpu::topk_select(logits, V, K, vals, ids); });
}

REF_API int ref_rep_penalties(float* logits, int V, const i32* hist, int hist_n, float rep,
                              float freq, float pres) {
    return guarded([&] { cpu::apply_rep_penalties(logits, V, hist, hist_n, rep, freq, pres); });
}

// wkind -2: fp32 experts (cpu::moe_forward_bias); -1: fp16 experts
// (cpu::moe_forward_bias_half); 0..2: packed experts materialised to fp16 through
// ops::quant_materialize exactly as inference/generator.cpp:274-285 does on CPU.
REF_API int ref_moe_forward(const float* x, const float* router_w, const float* router_bias,
                            const void* gates, const void* ups, const void* downs,
                            const void* sh_g, const void* sh_u, const void* sh_d, float* out,
                            float* probs_cache, i32* idx_cache, float* w_cache, i64 N, int d,
                            int E, int ne, int K, int SH, int wkind) {
    return guarded([&] {
        std::vector<float> sg(static_cast<size_t>(N) * K * E), su(sg.size()), sa(sg.size());
        if (wkind == -2) {
            cpu::moe_forward_bias(x, router_w, router_bias, static_cast<const float*>(gates),
                                  static_cast<const float*>(ups), static_cast<const float*>(downs),
                                  static_cast<const float*>(sh_g), static_cast<const float*>(sh_u),
                                  static_cast<const float*>(sh_d), out, probs_cache, idx_cache,
                                  w_cache, sg.data(), su.data(), sa.data(), N, d, E, ne, K, SH);
            return;
        }
        const u16 *g16, *u16p, *d16, *sg16 = nullptr, *su16 = nullptr, *sd16 = nullptr;
        if (wkind == -1) {
            g16 = static_cast<const u16*>(gates);
            u16p = static_cast<const u16*>(ups);
            d16 = static_cast<const u16*>(downs);
            sg16 = static_cast<const u16*>(sh_g);
            su16 = static_cast<const u16*>(sh_u);
            sd16 = static_cast<const u16*>(sh_d);
        } else {
            const i64 ne_w = static_cast<i64>(ne) * E * d;
            g16 = ops::quant_materialize(Device::CPU, gates, wkind, ne_w, 0);
            u16p = ops::quant_materialize(Device::CPU, ups, wkind, ne_w, 1);
            d16 = ops::quant_materialize(Device::CPU, downs, wkind, ne_w, 2);
            if (sh_g) sg16 = ops::quant_materialize(Device::CPU, sh_g, wkind, static_cast<i64>(SH) * d, 3);
            if (sh_u) su16 = ops::quant_materialize(Device::CPU, sh_u, wkind, static_cast<i64>(SH) * d, 4);
            if (sh_d) sd16 = ops::quant_materialize(Device::CPU, sh_d, wkind, static_cast<i64>(SH) * d, 5);
        }
        cpu::moe_forward_bias_half(x, router_w, router_bias, g16, u16p, d16, sg16, su16, sd16, out,
                                   probs_cache, idx_cache, w_cache, sg.data(), su.data(), sa.data(),
                                   N, d, E, ne, K, SH);
    });
}

// wkind -2 fp32 / -1 fp16 / 0..2 packed (materialised to fp16 like the CPU path
// of Model::forward_mamba_layer does through weight16()).
REF_API int ref_mamba2_forward(const float* x, const void* w_in, const float* conv_w,
                               const float* conv_b, const float* dt_bias, const float* a_log,
                               const float* Dv, const float* norm_w, const void* w_out,
                               float* state, float* out, int B, int T, int d, int d_inner,
                               int conv_dim, int n_heads, int d_head, int d_state, int k,
                               float eps, int wkind) {
    return guarded([&] {
        if (wkind == -2) {
            cpu::mamba2_forward(x, static_cast<const float*>(w_in), conv_w, conv_b, dt_bias, a_log,
                                Dv, norm_w, static_cast<const float*>(w_out), state, out, B, T, d,
                                d_inner, conv_dim, n_heads, d_head, d_state, k, eps);
            return;
        }
        const int proj = d_inner + conv_dim + n_heads;
        const u16 *wi, *wo;
        if (wkind == -1) {
            wi = static_cast<const u16*>(w_in);
            wo = static_cast<const u16*>(w_out);
        } else {
            wi = ops::quant_materialize(Device::CPU, w_in, wkind, static_cast<i64>(proj) * d, 0);
            wo = ops::quant_materialize(Device::CPU, w_out, wkind, static_cast<i64>(d) * d_inner, 1);
        }
        cpu::mamba2_forward_half(x, wi, conv_w, conv_b, dt_bias, a_log, Dv, norm_w, wo, state, out,
                                 B, T, d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps);
    });
}

REF_API int ref_attention_forward(const float* q, const float* k, const float* v, float* out,
                                  float* probs, int B, int T, int H, int KV, int hd, float scale,
                                  int window, const i32* segment_ids) {
    return guarded([&] {
        cpu::attention_forward_ex(q, k, v, out, probs, B, T, H, KV, hd, scale, window, segment_ids);
    });
}

REF_API int ref_attention_decode_ring(const float* q, const void* kc, const void* vc, int half,
                                      float* out, int H, int KV, int hd, int ring_start,
                                      int pinned, int cur_len, int cache_max, float scale,
                                      int window) {
    return guarded([&] {
        std::vector<float> scratch(static_cast<size_t>(H) * (cur_len > 0 ? cur_len : 1));
        if (half)
            cpu::attention_decode_ring_fp16(q, static_cast<const u16*>(kc),
                                            static_cast<const u16*>(vc), out, H, KV, hd, ring_start,
                                            pinned, cur_len, cache_max, scale, scratch.data(), window);
        else
            cpu::attention_decode_ring(q, static_cast<const float*>(kc),
                                       static_cast<const float*>(vc), out, H, KV, hd, ring_start,
                                       pinned, cur_len, cache_max, scale, scratch.data(), window);
    });
}
