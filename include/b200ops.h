/* b200ops - C ABI of the B200 (sm_100a) backend for the quantized hybrid-layer
 * forward step (Mamba-2 + GQA + MoE).
 *
 * Every entry point replaces one function of the reference engine's CUDA op API
 * (namespace gai::cuda_ops, cuda/cuda_ops.h, and gai::cuda, cuda/cuda_utils.h);
 * the reference declaration each one stands in for is cited beside it.  Argument
 * order and meaning are the reference's.  All tensor pointers are caller-owned
 * DEVICE memory unless a name ends in _host; nothing is retained after the call
 * returns (work is enqueued on the library's current stream, the legacy default
 * stream unless b200_set_stream() changed it).
 *
 * Errors: every function returns 0 on success and a negative B200_E* code
 * otherwise; b200_last_error() gives the message.  The library never aborts,
 * never traps a device and has no CPU fallback.
 *
 * Packed weight kinds ("qkind"/"kind"): 0 = Q4_0, 1 = Q4_1, 2 = Q8_0 (32-element
 * GGML blocks of 18/20/34 bytes, core/dtype.h:35-53), 3 = Q4_K (256-element
 * super-blocks of 144 bytes; an extension, the reference has no Q4_K), -1 = the
 * u16 pointer holds plain fp16 values.
 */
#ifndef B200OPS_H
#define B200OPS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK 0
#define B200_EINVAL (-1)      /* argument rejected (same checks as the reference's GAI_CHECKs) */
#define B200_ECUDA (-2)       /* a CUDA runtime call or launch failed */
#define B200_EUNSUPPORTED (-3)/* training-only op, not provided by this inference backend */
#define B200_ENOMEM (-4)

const char* b200_last_error(void);
int b200_version(void);
/* Kernels this library has enqueued so far in this process (a graph replay is not counted). */
uint64_t b200_kernel_launches(void);
/* Waits inside the TMA / tensor-core kernels are bounded: a kernel whose wait runs out
 * raises a device status word, skips its stores and returns.  This call synchronises the
 * device, reads the word back, clears it, and returns B200_OK or B200_ECUDA.  (The
 * reference has no such waits; b200_synchronize and b200_decoder_step_host check too.) */
int b200_stream_status(void);
/* Self-test of that mechanism: one kernel waits (at most spin_limit tries) on a barrier nobody
 * arrives on, gives up, raises the status word and returns; outcome_dev (device int) becomes 2
 * (1 would mean the wait was satisfied).  Enqueues only: read the word with b200_stream_status. */
int b200_test_bounded_wait(int spin_limit, int* outcome_dev);

/* ---- phase timers: cuda_ops.h:315-319 (phase_start / _stop / _reset / _shutdown / _report).
 * Event pairs recorded on the library's stream, never blocking the host; a start while a
 * phase is open closes that one first.  b200_phase_report adds, per phase id 0 .. n_phases-1
 * (n_phases <= 8), the milliseconds of the intervals that have completed since the last
 * report (intervals still running are kept for the next one).  The same ids also open and
 * close NVTX ranges ("b200.phase<id>") for timeline tools. */
int b200_phase_start(int phase);
int b200_phase_stop(int phase);
int b200_phase_reset(void);
int b200_phase_shutdown(void);
int b200_phase_report(double* ms_per_phase, int n_phases);

/* ---- device utilities: gai::cuda::*, cuda/cuda_utils.h:14-33 ------------------ */
int b200_device_count(int* count);                       /* probe(), :14 */
/* What probe() fills into gai::DeviceInfo (core/device.h): the current device
 * (LOCAL_RANK selects it on first use, as cuda/cuda_utils.cu:46-55 does). */
int b200_device_info(int* index, char* name, int name_cap, int* cc_major, int* cc_minor,
                     size_t* total_mem, size_t* free_mem);
int b200_shutdown(void);                                 /* shutdown(), :31: frees every cached workspace */
int b200_malloc_device(void** ptr, size_t nbytes);       /* malloc_device, :16 */
int b200_free_device(void* ptr);                         /* free_device, :17 */
int b200_memset_zero(void* ptr, size_t nbytes);          /* memset_zero, :18 */
int b200_is_device_memory(const void* ptr, int* yes);    /* is_device_memory, :20 */
int b200_copy(void* dst, int dst_is_device, const void* src, int src_is_device, size_t nbytes); /* copy, :21 */
int b200_synchronize(void);                              /* synchronize, :22 */
int b200_free_bytes_live(size_t* bytes);                 /* free_bytes_live, :24 */
/* Extension: the stream all later calls are enqueued on (a cudaStream_t; NULL =
 * the legacy default stream the reference uses everywhere). */
int b200_set_stream(void* cuda_stream);

/* ---- toggles: cuda/cuda_ops.h:14-21.  Accepted and recorded; the backend has one
 * arithmetic path (fp32 accumulate), so they do not change results. */
int b200_set_fp16_gemm(int on);
int b200_fp16_gemm_enabled(void);
int b200_set_bf16_gemm(int on);
int b200_bf16_gemm_enabled(void);
int b200_set_moe_jitter(float j);                        /* training-time router noise; must be 0 */
int b200_set_moe_jitter_seed(uint64_t seed);

/* ---- linear layers: y[M,N] = x[M,K] . W^T, W row-major [N,K] ------------------- */
int b200_linear_forward(const float* x, const float* w, float* y, int M, int K, int N);      /* cuda_ops.h:23 */
int b200_linear_forward_f32(const float* x, const float* w, float* y, int M, int K, int N);  /* :26 (router logits) */
int b200_linear_forward_fp16(const float* x, const uint16_t* w, float* y, int M, int K, int N); /* :27 */
int b200_linear_forward_q4(const float* x, const uint16_t* w, float* y, int M, int K, int N, int kind); /* :34 */
/* gemm(): cuda_ops.h:10.  Only the inference form (no transposes on A, B transposed,
 * alpha 1, beta 0) is provided; anything else returns B200_EUNSUPPORTED. */
int b200_gemm(int trans_a, int trans_b, int M, int N, int K, float alpha, const float* A, int lda,
              const float* B, int ldb, float beta, float* C, int ldc);
int b200_dequantize_quant(const uint16_t* src, uint16_t* dst, int64_t n, int kind);          /* :32 */
int b200_quant_scratch(int slot, int64_t n, uint16_t** out);                                 /* :39 */
int b200_free_quant_scratch(void);                                                           /* :40 */
int b200_split_qkv(const float* qkv, float* q, float* k, float* v, int64_t n, int qd, int kvd); /* :28 */
int b200_convert_f32_to_f16(const float* src, uint16_t* dst, int64_t n);                     /* :29 */
int b200_convert_f16_to_f32(const uint16_t* src, float* dst, int64_t n);                     /* :30 */

/* ---- elementwise: cuda_ops.h:64-70 --------------------------------------------- */
int b200_add(const float* a, const float* b, float* out, int64_t n);
int b200_add_inplace(float* a, const float* b, int64_t n);
int b200_add_bias(const float* b, float* y, int64_t rows, int cols);
int b200_scale_inplace(float* a, float s, int64_t n);
int b200_zero(float* a, int64_t n);
int b200_copy_f32(float* dst, const float* src, int64_t n);                                  /* copy(), :70 */

/* ---- embedding, norm, RoPE, SwiGLU: cuda_ops.h:72-97 ---------------------------- */
int b200_embedding_forward(const int32_t* ids, const float* table, float* out, int64_t ntok, int dim, int vocab);         /* :72 */
int b200_embedding_forward_half(const int32_t* ids, const uint16_t* table, float* out, int64_t ntok, int dim, int vocab); /* :74 */
int b200_rmsnorm_forward(const float* x, const float* weight, float* out, float* rrms, int64_t rows, int dim, float eps); /* :79; x may alias out */
int b200_rope_forward_cached(float* q, float* k, const int32_t* pos, const float* inv_freq, int64_t ntok,
                             int n_heads, int n_kv, int head_dim, int rope_type);                                          /* :92 */
int b200_swiglu_forward(const float* g, const float* u, float* out, int64_t n);                                           /* :97 */

/* ---- MoE: cuda_ops.h:101-130.  gates/ups [ne*E, d], downs [ne*d, E], shared
 * [SH,d],[SH,d],[d,SH] (NULL = no shared expert).  probs_cache [N,ne], idx_cache
 * [N,K], w_cache [N,K] and s_gate/s_up/s_act [N,K,E] are optional outputs (NULL
 * skips them).  The reference's limits ne <= 64, K <= 8 are lifted to ne <= 256,
 * K <= 16. */
int b200_moe_forward(const float* x, const float* router_w, const float* gates, const float* ups,
                     const float* downs, const float* sh_g, const float* sh_u, const float* sh_d,
                     float* out, float* probs_cache, int32_t* idx_cache, float* w_cache,
                     float* s_gate, float* s_up, float* s_act,
                     int64_t N, int d, int E, int ne, int K, int SH);                        /* :101 */
int b200_moe_forward_bias(const float* x, const float* router_w, const float* router_bias,
                          const float* gates, const float* ups, const float* downs,
                          const float* sh_g, const float* sh_u, const float* sh_d,
                          float* out, float* probs_cache, int32_t* idx_cache, float* w_cache,
                          float* s_gate, float* s_up, float* s_act,
                          int64_t N, int d, int E, int ne, int K, int SH);                   /* :108 */
int b200_moe_forward_half(const float* x, const float* router_w, const uint16_t* gates,
                          const uint16_t* ups, const uint16_t* downs, const uint16_t* sh_g,
                          const uint16_t* sh_u, const uint16_t* sh_d, float* out,
                          float* probs_cache, int32_t* idx_cache, float* w_cache,
                          float* s_gate, float* s_up, float* s_act,
                          int64_t N, int d, int E, int ne, int K, int SH, int qkind);        /* :117 */
int b200_moe_forward_bias_half(const float* x, const float* router_w, const float* router_bias,
                               const uint16_t* gates, const uint16_t* ups, const uint16_t* downs,
                               const uint16_t* sh_g, const uint16_t* sh_u, const uint16_t* sh_d,
                               float* out, float* probs_cache, int32_t* idx_cache, float* w_cache,
                               float* s_gate, float* s_up, float* s_act,
                               int64_t N, int d, int E, int ne, int K, int SH, int qkind);   /* :124 */
/* Extension (the reference keeps its grouping internal, cuda/moe.cu:623-651): the
 * expert permutation of the last routing - slot ids s = t*K+k stably sorted by
 * expert - and the exclusive prefix sums of the per-expert counts.
 * grouped [N*K] int32, offsets [ne+1] int32, both device pointers. */
int b200_moe_permutation(const int32_t* idx, int64_t NK, int ne, int32_t* grouped, int32_t* offsets);

/* Extensions for expert parallelism (the reference runs the MoE layer on one device
 * only): the layer cut at its two exchange points.  The caller - one process per GPU -
 * moves rows16 to the ranks that own the experts and y back, with any transport
 * (jdm-ghassan_v1_flach_b200/ep.py uses NCCL all-to-all through torch.distributed).
 * All pointers are device pointers; qkind -1 = fp16 experts, 0..3 packed (then d, E and
 * SH must be multiples of 256).
 *
 * route          probs [N,ne] (optional), idx [N,K], w [N,K]: the router alone, bit for
 *                bit the routing of b200_moe_forward_bias.
 * dispatch_pack  rows16 [N*K, d] fp16: the token row of every slot t*K+k, slots stably
 *                sorted by expert (so rows bound for one rank are contiguous);
 *                inv [N*K]: position of slot s in that order; offsets [ne+1].
 * experts_rows   y [R, d] fp32 = down_e(silu(gate_e r) * up_e r) for R received rows cut
 *                into `groups` consecutive blocks by offsets [groups+1]; block g uses
 *                local expert group_map[g] (null: g) of the n_local experts stored in
 *                gates/ups [n_local*E, d] and downs [n_local*d, E].
 * shared_combine out [N, d] = shared_expert(x) + sum_k w[t,k] * y[inv[t*K+k]] (k order);
 *                sh_* may be null (no shared expert). */
int b200_moe_route(const float* x, const float* router_w, const float* router_bias, float* probs, int32_t* idx,
                   float* w, int64_t N, int d, int ne, int K);
int b200_moe_dispatch_pack(const float* x, const int32_t* idx, int64_t N, int d, int ne, int K, uint16_t* rows16,
                           int32_t* inv, int32_t* offsets);
int b200_moe_experts_rows(const uint16_t* rows16, const int32_t* offsets, const int32_t* group_map, int groups,
                          int64_t R, const void* gates, const void* ups, const void* downs, int n_local, float* y,
                          int d, int E, int qkind);
int b200_moe_shared_combine(const float* x, const void* sh_g, const void* sh_u, const void* sh_d, const float* y,
                            const int32_t* inv, const float* w, float* out, int64_t N, int d, int K, int SH, int qkind);
/* The two halves of shared_combine, for callers that overlap the shared expert with the
 * exchange: out = shared_expert(x) (nothing when a matrix is null or SH == 0), then
 * out (+)= sum_k w[t,k] * y[inv[t*K+k]] (accumulate != 0: onto what out holds). */
int b200_moe_shared_expert(const float* x, const void* sh_g, const void* sh_u, const void* sh_d, float* out, int64_t N,
                           int d, int SH, int qkind);
int b200_moe_combine(const float* y, const int32_t* inv, const float* w, float* out, int64_t N, int d, int K,
                     int accumulate);

/* ---- Mamba-2: cuda_ops.h:142-189 ------------------------------------------------ */
int b200_mamba2_forward(const float* x, const float* w_in, const float* conv_w, const float* conv_b,
                        const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                        const float* w_out, float* state, float* out, int B, int T, int d, int d_inner,
                        int conv_dim, int n_heads, int d_head, int d_state, int k, float eps);              /* :142 */
int b200_mamba2_forward_half(const float* x, const uint16_t* w_in, const float* conv_w, const float* conv_b,
                             const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                             const uint16_t* w_out, float* state, float* out, int B, int T, int d, int d_inner,
                             int conv_dim, int n_heads, int d_head, int d_state, int k, float eps, int qkind); /* :160 */
int b200_mamba2_step(const float* x, const float* w_in, const float* conv_w, const float* conv_b,
                     const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                     const float* w_out, float* conv_state, float* ssm_state, float* out,
                     int d, int d_inner, int conv_dim, int n_heads, int d_head, int d_state, int k, float eps); /* :176 */
int b200_mamba2_step_half(const float* x, const uint16_t* w_in, const float* conv_w, const float* conv_b,
                          const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                          const uint16_t* w_out, float* conv_state, float* ssm_state, float* out,
                          int d, int d_inner, int conv_dim, int n_heads, int d_head, int d_state, int k,
                          float eps, int qkind);                                                              /* :183 */
/* Extension: the same step for `batch` independent sequences.  x/out [batch,d],
 * conv_state [batch, conv_dim, k-1], ssm_state [batch, n_heads*d_head, d_state]. */
int b200_mamba2_step_batched(const float* x, const uint16_t* w_in, const float* conv_w, const float* conv_b,
                             const float* dt_bias, const float* a_log, const float* D, const float* norm_w,
                             const uint16_t* w_out, float* conv_state, float* ssm_state, float* out,
                             int batch, int d, int d_inner, int conv_dim, int n_heads, int d_head,
                             int d_state, int k, float eps, int qkind);

/* ---- attention: cuda_ops.h:254-270 ---------------------------------------------- */
int b200_attention_forward_ex(const float* q, const float* k, const float* v, float* out, float* probs,
                              int B, int T, int H, int KV, int hd, float scale, int window,
                              const int32_t* segment_ids);                                   /* :254 */
int b200_attention_decode_ring(const float* q, const float* kcache, const float* vcache, float* out,
                               int H, int KV, int hd, int ring_start, int pinned_prefix, int cur_len,
                               int cache_max, float scale, float* scratch, int window);      /* :262 */
int b200_attention_decode_ring_fp16(const float* q, const uint16_t* kc, const uint16_t* vc, float* out,
                                    int H, int KV, int hd, int ring_start, int pinned_prefix, int cur_len,
                                    int cache_max, float scale, float* scratch, int window); /* :267 */
/* Extension: decode attention for `batch` ragged sequences over a paged fp16 KV
 * cache.  q/out [batch,H,hd]; k_pages/v_pages [num_pages, page, KV*hd] fp16;
 * page_table [batch, max_pages] int32 (page ids in logical order); seq_lens
 * [batch] int32 (tokens already in the cache, the new one included). */
int b200_attention_decode_paged_fp16(const float* q, const uint16_t* k_pages, const uint16_t* v_pages,
                                     const int32_t* page_table, const int32_t* seq_lens, float* out,
                                     int batch, int max_pages, int page, int H, int KV, int hd, float scale);
/* No counterpart in the reference.  b200_attention_decode_ring_fp16 for hosts that
 * must not allocate device memory on the decode path (an application that gave the
 * whole GPU to its own pool, a thread that cannot afford the device-wide
 * synchronisation of cudaMalloc/cudaFree, a process in which another thread is
 * capturing a stream).  The split-KV partial results go to a 1 MiB array built into
 * the library (resident on every GPU that loads it until the process exits) instead
 * of the growing workspace; the call performs no cudaMalloc / cudaFree and uses no
 * allocating library routine.  Limits: H * (hd + 2) <= 262144 floats, otherwise
 * B200_EINVAL with a message naming the allocating entry point.  The first call on
 * each device resolves the array's device address (make it before any stream
 * capture).  All calls share the one array, which keeps the previous call's partial
 * results (nothing in it has to start at zero: every record read is written first by
 * the same call); two calls whose kernels overlap on the GPU - different streams,
 * no ordering - race on it.  Same arguments as the ring fp16 entry point without
 * `scratch`. */
int b200_attention_decode_ring_fp16_noalloc(const float* q, const uint16_t* kc, const uint16_t* vc, float* out,
                                            int H, int KV, int hd, int ring_start, int pinned_prefix,
                                            int cur_len, int cache_max, float scale, int window);

/* ---- sampling tail: cuda_ops.h:289-293 ------------------------------------------ */
int b200_topk_select(const float* logits, int V, int K, float* out_vals, int32_t* out_ids);  /* :289; outputs on device */
/* cuda_ops.h:278, forward part (dlogits must be NULL: the gradient is a training op): sum over
 * rows with a target in [0, V) of logZ - logit[target] + z_scale * logZ^2, and their count;
 * host outputs, synchronises.  A negative target skips the row; a target >= V is an error. */
int b200_softmax_cross_entropy(const float* logits, const int32_t* targets, float* dlogits, int64_t n, int V,
                               double* out_loss_sum, int64_t* out_count, float z_scale);
int b200_argmax_token(const float* logits, int V, int32_t* token_host);                      /* :290; synchronous D2H */
int b200_argmax_token_device(const float* logits, int V, int32_t* token_dev);                /* extension: no sync */
/* :291.  hist: a host array as in the reference (staged to the device here), or a device pointer
 * (used in place). */
int b200_apply_rep_penalties(float* logits, int V, const int32_t* hist, int hist_n,
                             float rep, float freq, float pres);
int b200_free_sampling_workspace(void);                                                      /* :293 */

/* ---- workspaces: cuda_ops.h:157,309-328 ----------------------------------------- */
int b200_free_workspace(void);
int b200_moe_free_workspace(void);
int b200_mamba_free_workspace(void);
int b200_free_workspaces(void);
int b200_reserve_workspaces(size_t gemm_bytes, size_t moe_bytes);
int b200_moe_reserve_workspace(size_t bytes);
size_t b200_pool_bytes(void);
size_t b200_moe_pool_bytes(void);

/* ---- training-only ops of cuda_ops.h (backward passes, losses, optimizers, MoE
 * aux loss, rope_*_ex): not provided.  The C++ shim maps each of them to this. */
int b200_training_op_unsupported(const char* name);

#ifdef __cplusplus
}
#endif
#endif /* B200OPS_H */
