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

// ---------------------------------------------------------------------------
// Model level: the reference's own Model + Generator, unmodified, on the CPU device
// (libgai_ref.so) or - when this file is linked into libgai_b200.so with the
// reference compiled for GAI_CUDA and the B200 shim standing in for its CUDA
// backend - on the CUDA device.  Generator::decode_step_logits is private; the test
// bridge reaches it by including the header with private opened up.
// ---------------------------------------------------------------------------
#define private public
#include "inference/generator.h"
#undef private
#include "core/quant.h"
#include "model/model.h"
#include "tokenizer/tokenizer.h"

#include <memory>

namespace {
struct RefSession {
    ModelConfig cfg;
    std::unique_ptr<Model> model;
    Tokenizer tok;
    std::unique_ptr<Generator> gen;
};
}  // namespace

// icfg: vocab, hidden, n_layers, n_heads, n_kv, head_dim, rope_type(-1 none),
//       mamba_heads, mamba_d_head, mamba_d_state, mamba_d_conv, n_experts, top_k,
//       expert_dim, shared_dim, max_ctx
// fcfg: rope_theta, rms_eps, embedding_multiplier, residual_multiplier,
//       attention_multiplier, logits_scaling
// device: 0 CPU, 1 CUDA; quant_kind: -1 fp32 weights, 0..2 packed (fp16 embeddings)
REF_API void* ref_model_create(const int* icfg, const float* fcfg, const int* layer_types, int device,
                               int quant_kind) {
    RefSession* s = new RefSession();
    try {
        ModelConfig& c = s->cfg;
        c.arch = ModelConfig::ArchGranite;
        c.vocab_size = icfg[0]; c.hidden_size = icfg[1]; c.num_layers = icfg[2];
        c.num_heads = icfg[3]; c.num_kv_heads = icfg[4]; c.head_dim_override = icfg[5];
        c.position_embedding = icfg[6] < 0 ? 1 : 0;
        c.rope_type = icfg[6] < 0 ? 1 : icfg[6];
        c.mamba_n_heads = icfg[7]; c.mamba_d_head = icfg[8]; c.mamba_d_state = icfg[9]; c.mamba_d_conv = icfg[10];
        c.mamba_n_groups = 1;
        c.mamba_expand = (icfg[7] * icfg[8]) / icfg[1];
        c.use_moe = true; c.num_experts = icfg[11]; c.moe_top_k = icfg[12]; c.moe_expert_dim = icfg[13];
        c.moe_shared = icfg[14] > 0; c.shared_expert_intermediate_size = icfg[14];
        c.max_seq_len = icfg[15];
        c.tie_embeddings = true;
        c.rope_theta = fcfg[0]; c.rms_eps = fcfg[1]; c.embedding_multiplier = fcfg[2];
        c.residual_multiplier = fcfg[3]; c.attention_multiplier = fcfg[4]; c.logits_scaling = fcfg[5];
        c.layer_types.assign(layer_types, layer_types + c.num_layers);
        c.validate();
        s->model.reset(new Model(c, device ? Device::CUDA : Device::CPU, false, quant_kind));
    } catch (const std::exception& e) {
        g_err = e.what();
        delete s;
        return nullptr;
    }
    return s;
}

REF_API void ref_model_destroy(void* h) { delete static_cast<RefSession*>(h); }

REF_API int ref_model_param_count(void* h) {
    return static_cast<int>(static_cast<RefSession*>(h)->model->parameters().size());
}

// name, element count and storage dtype code (DType) of parameter i
REF_API int ref_model_param_info(void* h, int i, char* name, int cap, i64* numel, int* dtype) {
    return guarded([&] {
        Parameter* p = static_cast<RefSession*>(h)->model->parameters().at(static_cast<size_t>(i));
        std::snprintf(name, static_cast<size_t>(cap), "%s", p->name.c_str());
        *numel = p->w.numel();
        *dtype = static_cast<int>(p->w.dtype());
    });
}

// Fill a parameter from fp32 host data the way load-time quantisation does
// (format/gguf_codec.cpp:1495-1500): packed tensors through quant::quantize, fp16
// tensors through copy_from_f32, fp32 tensors verbatim.
REF_API int ref_model_set_param(void* h, const char* name, const float* data, i64 n) {
    return guarded([&] {
        RefSession* s = static_cast<RefSession*>(h);
        Parameter* p = s->model->find_parameter(name);
        GAI_CHECK(p != nullptr, std::string("no such parameter: ") + name);
        GAI_CHECK(p->w.numel() == n, std::string("element count mismatch for ") + name);
        Tensor src(p->shape, DType::F32, Device::CPU);
        std::memcpy(src.data_ptr(), data, sizeof(float) * static_cast<size_t>(n));
        if (is_quant(p->w)) p->w.copy_from(quant::quantize(src, p->w.dtype()));
        else if (p->w.dtype() == DType::F16) p->w.copy_from_f32(src);
        else p->w.copy_from(src);
    });
}

REF_API int ref_generator_create(void* h, int max_ctx) {
    return guarded([&] {
        RefSession* s = static_cast<RefSession*>(h);
        s->model->rebuild_rope_cache();
        s->gen.reset(new Generator(*s->model, s->tok, max_ctx));
        s->gen->reset();
    });
}

REF_API int ref_generator_reset(void* h) {
    return guarded([&] { static_cast<RefSession*>(h)->gen->reset(); });
}

// One token through Generator::decode_step (logits copied to the host).
REF_API int ref_decode_step(void* h, int token, int position, float* logits_out) {
    return guarded([&] {
        RefSession* s = static_cast<RefSession*>(h);
        const float* lp = s->gen->decode_step(token, position);
        std::memcpy(logits_out, lp, sizeof(float) * static_cast<size_t>(s->cfg.vocab_size));
    });
}

// ---------------------------------------------------------------------------
// GGUF: the reference's own writer and reader (format/gguf_codec.cpp).  Used to make
// the committed fixture tests/golden/tiny.gguf and to check the device loader against
// GGUFReader::read_tensor_quant / read_tensor_f32.
// ---------------------------------------------------------------------------
#include "format/gguf_codec.h"

// n two-dimensional fp32 tensors [rows, cols] (cols == 0: one-dimensional [rows]) written in
// the given GGML types by GGUFWriter.
REF_API int ref_gguf_write(const char* path, int n, const char* const* names, const i64* rows, const i64* cols,
                           const float* const* data, const int* ggml_types) {
    return guarded([&] {
        GGUFWriter w(path);
        w.set_arch("granitehybrid");
        w.set_model_name("b200-fixture");
        w.set_hidden_size(64);
        w.set_num_layers(1);
        w.set_rms_eps(1e-5f);
        w.add_custom_metadata("b200.fixture.answer", static_cast<uint64_t>(42));
        for (int i = 0; i < n; ++i) {
            std::vector<i64> shape = cols[i] > 0 ? std::vector<i64>{rows[i], cols[i]} : std::vector<i64>{rows[i]};
            Tensor t(shape, DType::F32, Device::CPU);
            std::memcpy(t.data_ptr(), data[i], sizeof(float) * static_cast<size_t>(t.numel()));
            w.add_tensor(names[i], t, static_cast<GGMLType>(ggml_types[i]));
        }
        w.write();
    });
}

// kind: 0 Q4_0, 1 Q4_1, 2 Q8_0 (read_tensor_quant: verbatim blocks or quantise on load); -2: fp32
REF_API int ref_gguf_read(const char* path, const char* name, int kind, void* out, i64 cap, i64* nbytes) {
    return guarded([&] {
        GGUFReader r;
        GAI_CHECK(r.open(path), std::string("cannot open ") + path);
        Tensor t = kind == -2 ? r.read_tensor_f32(name)
                              : r.read_tensor_quant(name, kind == 0 ? DType::Q4_0 : kind == 1 ? DType::Q4_1 : DType::Q8_0);
        GAI_CHECK(static_cast<i64>(t.nbytes()) <= cap, "output buffer too small");
        std::memcpy(out, t.data_ptr(), t.nbytes());
        *nbytes = static_cast<i64>(t.nbytes());
    });
}

// ---------------------------------------------------------------------------
// Sampling tail: the reference's Sampler (inference/sampler.cpp), its generator
// (core/rng.h) and the cross-entropy behind Generator::score_tokens.
// ---------------------------------------------------------------------------
#include "inference/sampler.h"

static SamplingConfig sampling_of(const float* f, const int* ic, u64 seed) {
    SamplingConfig c;
    c.temperature = f[0]; c.top_p = f[1]; c.min_p = f[2]; c.repetition_penalty = f[3];
    c.frequency_penalty = f[4]; c.presence_penalty = f[5];
    c.top_k = ic[0]; c.repetition_window = ic[1]; c.no_repeat_ngram = ic[2]; c.greedy = ic[3] != 0;
    c.seed = seed;
    return c;
}

// SamplingConfig::validate on the same packed fields.
REF_API int ref_sampling_validate(float* f, int* ic) {
    return guarded([&] {
        SamplingConfig c = sampling_of(f, ic, 1);
        c.validate();
        f[0] = c.temperature; f[1] = c.top_p; f[2] = c.min_p; f[3] = c.repetition_penalty;
        f[4] = c.frequency_penalty; f[5] = c.presence_penalty;
        ic[0] = c.top_k; ic[1] = c.repetition_window; ic[2] = c.no_repeat_ngram; ic[3] = c.greedy ? 1 : 0;
    });
}

// n_draws calls of Sampler::sample on fresh copies of the same logits (one Sampler, so the
// generator runs on from draw to draw).
REF_API int ref_sampler_sample(const float* logits, int V, const i32* hist, int nh, const float* f, const int* ic,
                               u64 seed, int n_draws, i32* out) {
    return guarded([&] {
        Sampler s(sampling_of(f, ic, seed));
        std::vector<i32> h(hist, hist + nh);
        std::vector<float> work(static_cast<size_t>(V));
        for (int i = 0; i < n_draws; ++i) {
            std::memcpy(work.data(), logits, sizeof(float) * static_cast<size_t>(V));
            out[i] = s.sample(work.data(), V, h);
        }
    });
}

REF_API int ref_sampler_candidates(const float* vals, const i32* ids, int K, const float* f, const int* ic, u64 seed,
                                   int n_draws, i32* out) {
    return guarded([&] {
        Sampler s(sampling_of(f, ic, seed));
        for (int i = 0; i < n_draws; ++i) out[i] = s.sample_candidates(vals, ids, K);
    });
}

REF_API int ref_rng_uniform(u64 seed, int n, float* out) {
    return guarded([&] {
        Rng r(seed);
        for (int i = 0; i < n; ++i) out[i] = r.uniform();
    });
}

REF_API int ref_softmax_cross_entropy(const float* logits, const i32* targets, i64 n, int V, float z_scale,
                                      double* loss_sum, i64* count) {
    return guarded([&] { cpu::softmax_cross_entropy(logits, targets, nullptr, n, V, loss_sum, count, z_scale); });
}

// Generator::score_tokens (inference/generator.cpp:1217-1294): mean negative log-likelihood.
REF_API int ref_score_tokens(void* h, const i32* tokens, int T, const unsigned char* mask, double* mean_nll,
                             i64* n_scored) {
    return guarded([&] {
        RefSession* s = static_cast<RefSession*>(h);
        std::vector<i32> t(tokens, tokens + T);
        std::vector<u8> m;
        if (mask) m.assign(mask, mask + T);
        *mean_nll = s->gen->score_tokens(t, mask ? &m : nullptr, n_scored, nullptr);
    });
}

// Generator::prefill + Generator::generate (inference/generator.cpp:917-1098) with a sampling
// configuration: on the CUDA device this is the engine's fast path (penalties and top-K on the
// device, Sampler::sample_candidates on the host), on the CPU device Sampler::sample.
REF_API int ref_generate(void* h, const i32* prompt, int n_prompt, int max_new, const float* f, const int* ic, u64 seed,
                         i32* out, int* n_out) {
    return guarded([&] {
        RefSession* s = static_cast<RefSession*>(h);
        s->gen->reset();
        s->gen->prefill(std::vector<i32>(prompt, prompt + n_prompt));
        GenerationConfig cfg;
        cfg.max_new_tokens = max_new;
        cfg.stop_tokens = {-1};
        cfg.sampling = sampling_of(f, ic, seed);
        const std::vector<i32> toks = s->gen->generate(cfg, nullptr);
        *n_out = static_cast<int>(toks.size());
        std::memcpy(out, toks.data(), sizeof(i32) * toks.size());
    });
}
