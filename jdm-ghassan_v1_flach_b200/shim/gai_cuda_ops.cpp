// Drop-in replacement for the reference engine's CUDA backend library (gai_cuda):
// defines every function of namespace gai::cuda_ops (cuda/cuda_ops.h) and
// gai::cuda (cuda/cuda_utils.h) with the reference's exact C++ signatures and
// forwards to the C ABI of libb200ops (include/b200ops.h).  A non-zero status
// becomes the reference's error convention: GAI_FAIL -> gai::Error.
//
// Build: compiled against the reference's own headers (-I<reference root>), with
// -DGAI_CUDA, then linked with gai_core in place of gai_cuda; model/model.cpp,
// inference/generator.cpp and inference/kv_cache.cpp are used unmodified.
// Training-only entry points (backward passes, losses, optimizers, MoE auxiliary
// loss, rope_*_ex) link but fail loudly when called.
#include "cuda/cuda_ops.h"
#include "cuda/cuda_utils.h"
#include "core/device.h"

#include <cstdio>
#include <string>

#include "b200ops.h"

namespace {
[[noreturn]] void raise(const char* op) {
    GAI_FAIL(std::string(op) + ": " + b200_last_error());
}
inline void ck(int rc, const char* op) {
    if (rc != B200_OK) raise(op);
}
[[noreturn]] void training(const char* op) {
    b200_training_op_unsupported(op);
    raise(op);
}
}  // namespace

namespace gai {

// ---------------------------------------------------------------------------
// gai::cuda  (cuda/cuda_utils.h:14-33)
// ---------------------------------------------------------------------------
namespace cuda {

void probe(DeviceInfo& info) {
    int count = 0;
    if (b200_device_count(&count) != B200_OK || count <= 0) {
        info.cuda_available = false;
        return;
    }
    char name[256] = "";
    int index = 0, major = 0, minor = 0;
    size_t total = 0, free_b = 0;
    if (b200_device_info(&index, name, (int)sizeof(name), &major, &minor, &total, &free_b) != B200_OK) {
        info.cuda_available = false;
        return;
    }
    info.cuda_available = true;
    info.device_count = count;
    info.device_index = index;
    info.name = name;
    info.cc_major = major;
    info.cc_minor = minor;
    info.total_mem = total;
    info.free_mem = free_b;
    info.supports_fp16 = true;
    info.supports_bf16 = major >= 8;
    info.supports_tf32 = major >= 8;
}

void* malloc_device(size_t nbytes) {
    void* p = nullptr;
    ck(b200_malloc_device(&p, nbytes), "cuda::malloc_device");
    return p;
}
void free_device(void* ptr) { ck(b200_free_device(ptr), "cuda::free_device"); }
void memset_zero(void* ptr, size_t nbytes) { ck(b200_memset_zero(ptr, nbytes), "cuda::memset_zero"); }
bool is_device_memory(const void* ptr) {
    int yes = 0;
    ck(b200_is_device_memory(ptr, &yes), "cuda::is_device_memory");
    return yes != 0;
}
void copy(void* dst, bool dst_is_device, const void* src, bool src_is_device, size_t nbytes) {
    ck(b200_copy(dst, dst_is_device ? 1 : 0, src, src_is_device ? 1 : 0, nbytes), "cuda::copy");
}
void synchronize() { ck(b200_synchronize(), "cuda::synchronize"); }
size_t free_bytes_live() {
    size_t b = 0;
    ck(b200_free_bytes_live(&b), "cuda::free_bytes_live");
    return b;
}
void check_free_vram(size_t need, const char* what) {
    const size_t have = free_bytes_live();
    if (have < need)
        GAI_FAIL(std::string("not enough free device memory for ") + (what ? what : "allocation") + ": need " +
                 std::to_string(need) + " bytes, have " + std::to_string(have));
}
// The backend has no cuBLAS: callers that only pass the handle around get null.
void* cublas_handle() { return nullptr; }
int cublas_device() {
    int index = 0;
    b200_device_info(&index, nullptr, 0, nullptr, nullptr, nullptr, nullptr);
    return index;
}
void shutdown() { b200_shutdown(); }
const char* last_error() { return b200_last_error(); }

}  // namespace cuda

// ---------------------------------------------------------------------------
// gai::cuda_ops  (cuda/cuda_ops.h)
// ---------------------------------------------------------------------------
namespace cuda_ops {

void gemm(bool trans_a, bool trans_b, int M, int N, int K, float alpha, const float* A, int lda,
          const float* B, int ldb, float beta, float* C, int ldc, bool) {
    ck(b200_gemm(trans_a, trans_b, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc), "gemm");
}
void set_fp16_gemm(bool on) { b200_set_fp16_gemm(on); }
bool fp16_gemm_enabled() { return b200_fp16_gemm_enabled() != 0; }
void set_bf16_gemm(bool on) { b200_set_bf16_gemm(on); }
bool bf16_gemm_enabled() { return b200_bf16_gemm_enabled() != 0; }
void set_moe_jitter(float j) { ck(b200_set_moe_jitter(j), "set_moe_jitter"); }
void set_moe_jitter_seed(u64 seed) { b200_set_moe_jitter_seed(seed); }

void linear_forward(const float* x, const float* w, float* y, int M, int K, int N) {
    ck(b200_linear_forward(x, w, y, M, K, N), "linear_forward");
}
void linear_forward_f32(const float* x, const float* w, float* y, int M, int K, int N) {
    ck(b200_linear_forward_f32(x, w, y, M, K, N), "linear_forward_f32");
}
void linear_forward_fp16(const float* x, const u16* w, float* y, int M, int K, int N) {
    ck(b200_linear_forward_fp16(x, w, y, M, K, N), "linear_forward_fp16");
}
void split_qkv(const float* qkv, float* q, float* k, float* v, i64 n, int qd, int kvd) {
    ck(b200_split_qkv(qkv, q, k, v, n, qd, kvd), "split_qkv");
}
void convert_f32_to_f16(const float* src, u16* dst, i64 n) { ck(b200_convert_f32_to_f16(src, dst, n), "convert_f32_to_f16"); }
void convert_f16_to_f32(const u16* src, float* dst, i64 n) { ck(b200_convert_f16_to_f32(src, dst, n), "convert_f16_to_f32"); }
void dequantize_quant(const u16* src, u16* dst, i64 n, int kind) { ck(b200_dequantize_quant(src, dst, n, kind), "dequantize_quant"); }
void linear_forward_q4(const float* x, const u16* w, float* y, int M, int K, int N, int kind) {
    ck(b200_linear_forward_q4(x, w, y, M, K, N, kind), "linear_forward_q4");
}
u16* quant_scratch(int slot, i64 n) {
    u16* p = nullptr;
    ck(b200_quant_scratch(slot, n, &p), "quant_scratch");
    return p;
}
void free_quant_scratch() { b200_free_quant_scratch(); }

void add(const float* a, const float* b, float* out, i64 n) { ck(b200_add(a, b, out, n), "add"); }
void add_inplace(float* a, const float* b, i64 n) { ck(b200_add_inplace(a, b, n), "add_inplace"); }
void add_bias(const float* b, float* y, i64 rows, int cols) { ck(b200_add_bias(b, y, rows, cols), "add_bias"); }
void scale_inplace(float* a, float s, i64 n) { ck(b200_scale_inplace(a, s, n), "scale_inplace"); }
void zero(float* a, i64 n) { ck(b200_zero(a, n), "zero"); }
void copy(float* dst, const float* src, i64 n) { ck(b200_copy_f32(dst, src, n), "copy"); }

void embedding_forward(const i32* ids, const float* table, float* out, i64 ntok, int dim, int vocab) {
    ck(b200_embedding_forward(ids, table, out, ntok, dim, vocab), "embedding_forward");
}
void embedding_forward_half(const i32* ids, const u16* table, float* out, i64 ntok, int dim, int vocab) {
    ck(b200_embedding_forward_half(ids, table, out, ntok, dim, vocab), "embedding_forward_half");
}
void rmsnorm_forward(const float* x, const float* weight, float* out, float* rrms, i64 rows, int dim, float eps) {
    ck(b200_rmsnorm_forward(x, weight, out, rrms, rows, dim, eps), "rmsnorm_forward");
}
void rope_forward_cached(float* q, float* k, const i32* pos, const float* inv_freq, i64 ntok, int n_heads,
                         int n_kv, int head_dim, int rope_type) {
    ck(b200_rope_forward_cached(q, k, pos, inv_freq, ntok, n_heads, n_kv, head_dim, rope_type), "rope_forward_cached");
}
void swiglu_forward(const float* g, const float* u, float* out, i64 n) { ck(b200_swiglu_forward(g, u, out, n), "swiglu_forward"); }

void moe_forward(const float* x, const float* router_w, const float* gates, const float* ups, const float* downs,
                 const float* sh_g, const float* sh_u, const float* sh_d, float* out, float* probs_cache,
                 i32* idx_cache, float* w_cache, float* s_gate, float* s_up, float* s_act, i64 N, int d, int E,
                 int ne, int K, int SH) {
    ck(b200_moe_forward(x, router_w, gates, ups, downs, sh_g, sh_u, sh_d, out, probs_cache, idx_cache, w_cache,
                        s_gate, s_up, s_act, N, d, E, ne, K, SH), "moe_forward");
}
void moe_forward_bias(const float* x, const float* router_w, const float* router_bias, const float* gates,
                      const float* ups, const float* downs, const float* sh_g, const float* sh_u,
                      const float* sh_d, float* out, float* probs_cache, i32* idx_cache, float* w_cache,
                      float* s_gate, float* s_up, float* s_act, i64 N, int d, int E, int ne, int K, int SH) {
    ck(b200_moe_forward_bias(x, router_w, router_bias, gates, ups, downs, sh_g, sh_u, sh_d, out, probs_cache,
                             idx_cache, w_cache, s_gate, s_up, s_act, N, d, E, ne, K, SH), "moe_forward_bias");
}
void moe_forward_half(const float* x, const float* router_w, const u16* gates, const u16* ups, const u16* downs,
                      const u16* sh_g, const u16* sh_u, const u16* sh_d, float* out, float* probs_cache,
                      i32* idx_cache, float* w_cache, float* s_gate, float* s_up, float* s_act, i64 N, int d,
                      int E, int ne, int K, int SH, int qkind) {
    ck(b200_moe_forward_half(x, router_w, gates, ups, downs, sh_g, sh_u, sh_d, out, probs_cache, idx_cache,
                             w_cache, s_gate, s_up, s_act, N, d, E, ne, K, SH, qkind), "moe_forward_half");
}
void moe_forward_bias_half(const float* x, const float* router_w, const float* router_bias, const u16* gates,
                           const u16* ups, const u16* downs, const u16* sh_g, const u16* sh_u, const u16* sh_d,
                           float* out, float* probs_cache, i32* idx_cache, float* w_cache, float* s_gate,
                           float* s_up, float* s_act, i64 N, int d, int E, int ne, int K, int SH, int qkind) {
    ck(b200_moe_forward_bias_half(x, router_w, router_bias, gates, ups, downs, sh_g, sh_u, sh_d, out, probs_cache,
                                  idx_cache, w_cache, s_gate, s_up, s_act, N, d, E, ne, K, SH, qkind),
       "moe_forward_bias_half");
}

void mamba2_forward(const float* x, const float* w_in, const float* conv_w, const float* conv_b,
                    const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                    const float* w_out, float* state, float* out, int B, int T, int d, int d_inner, int conv_dim,
                    int n_heads, int d_head, int d_state, int k, float eps) {
    ck(b200_mamba2_forward(x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, state, out, B, T, d, d_inner,
                           conv_dim, n_heads, d_head, d_state, k, eps), "mamba2_forward");
}
void mamba_free_workspace() { b200_mamba_free_workspace(); }
void mamba2_forward_half(const float* x, const u16* w_in, const float* conv_w, const float* conv_b,
                         const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                         const u16* w_out, float* state, float* out, int B, int T, int d, int d_inner,
                         int conv_dim, int n_heads, int d_head, int d_state, int k, float eps, int qkind) {
    ck(b200_mamba2_forward_half(x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, state, out, B, T, d,
                                d_inner, conv_dim, n_heads, d_head, d_state, k, eps, qkind), "mamba2_forward_half");
}
void mamba2_step(const float* x, const float* w_in, const float* conv_w, const float* conv_b, const float* dt_bias,
                 const float* a_log, const float* D, const float* norm_w, const float* w_out, float* conv_state,
                 float* ssm_state, float* out, int d, int d_inner, int conv_dim, int n_heads, int d_head,
                 int d_state, int k, float eps) {
    ck(b200_mamba2_step(x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, conv_state, ssm_state, out, d,
                        d_inner, conv_dim, n_heads, d_head, d_state, k, eps), "mamba2_step");
}
void mamba2_step_half(const float* x, const u16* w_in, const float* conv_w, const float* conv_b,
                      const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                      const u16* w_out, float* conv_state, float* ssm_state, float* out, int d, int d_inner,
                      int conv_dim, int n_heads, int d_head, int d_state, int k, float eps, int qkind) {
    ck(b200_mamba2_step_half(x, w_in, conv_w, conv_b, dt_bias, a_log, D, norm_w, w_out, conv_state, ssm_state, out,
                             d, d_inner, conv_dim, n_heads, d_head, d_state, k, eps, qkind), "mamba2_step_half");
}

void attention_forward_ex(const float* q, const float* k, const float* v, float* out, float* probs, int B, int T,
                          int H, int KV, int hd, float scale, int window, const i32* segment_ids) {
    ck(b200_attention_forward_ex(q, k, v, out, probs, B, T, H, KV, hd, scale, window, segment_ids),
       "attention_forward_ex");
}
void attention_decode_ring(const float* q, const float* kcache, const float* vcache, float* out, int H, int KV,
                           int hd, int ring_start, int pinned_prefix, int cur_len, int cache_max, float scale,
                           float* scratch, int window) {
    ck(b200_attention_decode_ring(q, kcache, vcache, out, H, KV, hd, ring_start, pinned_prefix, cur_len, cache_max,
                                  scale, scratch, window), "attention_decode_ring");
}
void attention_decode_ring_fp16(const float* q, const u16* kc, const u16* vc, float* out, int H, int KV, int hd,
                                int ring_start, int pinned_prefix, int cur_len, int cache_max, float scale,
                                float* scratch, int window) {
    ck(b200_attention_decode_ring_fp16(q, kc, vc, out, H, KV, hd, ring_start, pinned_prefix, cur_len, cache_max,
                                       scale, scratch, window), "attention_decode_ring_fp16");
}

void topk_select(const float* logits, int V, int K, float* out_vals, i32* out_ids) {
    ck(b200_topk_select(logits, V, K, out_vals, out_ids), "topk_select");
}
i32 argmax_token(const float* logits, int V) {
    i32 tok = 0;
    ck(b200_argmax_token(logits, V, &tok), "argmax_token");
    return tok;
}
void apply_rep_penalties(float* logits, int V, const i32* hist, int hist_n, float rep, float freq, float pres) {
    ck(b200_apply_rep_penalties(logits, V, hist, hist_n, rep, freq, pres), "apply_rep_penalties");
}
void free_sampling_workspace() { b200_free_sampling_workspace(); }

void free_workspace() { b200_free_workspace(); }
void moe_free_workspace() { b200_moe_free_workspace(); }
void free_workspaces() { b200_free_workspaces(); }
void reserve_workspaces(size_t gemm_bytes, size_t moe_bytes) { ck(b200_reserve_workspaces(gemm_bytes, moe_bytes), "reserve_workspaces"); }
void moe_reserve_workspace(size_t bytes) { ck(b200_moe_reserve_workspace(bytes), "moe_reserve_workspace"); }
size_t pool_bytes() { return b200_pool_bytes(); }
size_t moe_pool_bytes() { return b200_moe_pool_bytes(); }

// Phase timers (cuda/cuda_utils.cu:200-288): event pairs on the library's stream.
void phase_start(int ph) { ck(b200_phase_start(ph), "phase_start"); }
void phase_stop(int ph) { ck(b200_phase_stop(ph), "phase_stop"); }
void phase_reset() { ck(b200_phase_reset(), "phase_reset"); }
void phase_shutdown() { ck(b200_phase_shutdown(), "phase_shutdown"); }
std::string phase_report() {
    // the reference's line: totals per TrainPhase since the last report (cuda/cuda_utils.cu:261-296)
    double ms[5] = {};
    ck(b200_phase_report(ms, 5), "phase_report");
    char buf[256];
    std::snprintf(buf, sizeof(buf), "ph [attnF %.1f moeF %.1f attnB %.1f moeB %.1f load %.1f]", ms[0], ms[1], ms[2], ms[3],
                  ms[4]);
    return std::string(buf);
}

// ---- training-only entry points: link, fail loudly --------------------------
void moe_backward_half(const float*, const float*, const u16*, const u16*, const u16*, const u16*, const u16*,
                       const u16*, const float*, const i32*, const float*, const float*, const float*, const float*,
                       const float*, float, const float*, float*, float*, float*, float*, float*, float*, float*,
                       float*, float*, i64, int, int, int, int, int) { training("moe_backward_half"); }
void moe_backward(const float*, const float*, const float*, const float*, const float*, const float*, const float*,
                  const float*, const float*, const i32*, const float*, const float*, const float*, const float*,
                  const float*, float, const float*, float*, float*, float*, float*, float*, float*, float*, float*,
                  float*, i64, int, int, int, int, int) { training("moe_backward"); }
void linear_backward(const float*, const float*, const float*, float*, float*, int, int, int) { training("linear_backward"); }
void gemm_nn_half(const float*, const u16*, float*, int, int, int) { training("gemm_nn_half"); }
void linear_backward_half(const float*, const u16*, const float*, float*, float*, int, int, int) { training("linear_backward_half"); }
void bias_backward(const float*, float*, i64, int) { training("bias_backward"); }
void embedding_backward(const i32*, const float*, float*, i64, int, int) { training("embedding_backward"); }
void rmsnorm_backward(const float*, const float*, const float*, const float*, float*, float*, i64, int) { training("rmsnorm_backward"); }
void rope_backward(float*, float*, const i32*, i64, int, int, int, float) { training("rope_backward"); }
void rope_forward_ex(float*, float*, const i32*, i64, int, int, int, float, int, float, float, float) { training("rope_forward_ex"); }
void rope_backward_ex(float*, float*, const i32*, i64, int, int, int, float, int, float, float, float) { training("rope_backward_ex"); }
void rope_backward_cached(float*, float*, const i32*, const float*, i64, int, int, int, int) { training("rope_backward_cached"); }
void swiglu_backward(const float*, const float*, const float*, float*, float*, i64) { training("swiglu_backward"); }
void mamba2_backward_half(const float*, const u16*, const float*, const float*, const float*, const float*,
                          const float*, const float*, const u16*, const float*, float*, float*, float*, float*,
                          float*, float*, float*, float*, float*, float*, int, int, int, int, int, int, int, int, int,
                          float) { training("mamba2_backward_half"); }
void mamba2_backward(const float*, const float*, const float*, const float*, const float*, const float*, const float*,
                     const float*, const float*, const float*, float*, float*, float*, float*, float*, float*, float*,
                     float*, float*, float*, int, int, int, int, int, int, int, int, int, float) { training("mamba2_backward"); }
void attention_backward_ex(const float*, const float*, const float*, const float*, const float*, float*, float*,
                           float*, int, int, int, int, int, float, int) { training("attention_backward_ex"); }
void moe_aux_frac_gpu(const float*, const i32*, float*, float*, float*, i64, int, int, double*) { training("moe_aux_frac_gpu"); }
double* moe_aux_begin() { training("moe_aux_begin"); }
double moe_aux_end() { training("moe_aux_end"); }
// The loss value alone (dlogits == nullptr) is what Generator::score_tokens asks for; with a
// gradient buffer it is a training call.
void softmax_cross_entropy(const float* logits, const i32* targets, float* dlogits, i64 n, int V, double* out_loss_sum,
                           i64* out_count, float z_scale) {
    if (dlogits) training("softmax_cross_entropy (with gradient)");
    int64_t count = 0;
    ck(b200_softmax_cross_entropy(logits, targets, nullptr, n, V, out_loss_sum, &count, z_scale), "softmax_cross_entropy");
    if (out_count) *out_count = count;
}
void sce_acc_begin() { training("sce_acc_begin"); }
void sce_accumulate(const float*, const i32*, float*, i64, int, float) { training("sce_accumulate"); }
void sce_acc_end(double*, i64*) { training("sce_acc_end"); }
void moe_count_slots(const i32*, float*, i64, int) { training("moe_count_slots"); }
void adamw_step(float*, const float*, float*, float*, i64, float, float, float, float, float, float, float, float) { training("adamw_step"); }
void lion_step(float*, const float*, float*, i64, float, float, float, float, float) { training("lion_step"); }
void scale_grad(float*, i64, float) { training("scale_grad"); }
double global_sq_norm(const float*, i64) { training("global_sq_norm"); }
double global_sq_norm_multi(const std::vector<std::pair<const float*, i64>>&) { training("global_sq_norm_multi"); }

}  // namespace cuda_ops
}  // namespace gai
