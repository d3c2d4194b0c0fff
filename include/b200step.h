/* b200step - whole-token decode step over the op library.
 *
 * The reference engine drives one token through the model with one op call at a
 * time (Generator::decode_step_logits, inference/generator.cpp:221-443, and
 * Generator::decode_mamba_layer, :456-617), copies the token id to the device and
 * the arg-max back per token, and keeps per-sequence state in Generator
 * (MambaState, generator.h:126-134; KVCache, inference/kv_cache.h:11-138).  A
 * b200_decoder holds the same state for `batch` independent sequences and
 * enqueues the same op sequence without any host synchronisation, so the whole
 * step can be replayed as one CUDA graph.
 *
 * Weights stay caller-owned device memory (like the reference's Model tensors):
 * the decoder only records the pointers given to b200_decoder_set_tensor.
 */
#ifndef B200STEP_H
#define B200STEP_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Tensor ids for b200_decoder_set_tensor.  Layer tensors take the layer index,
 * model tensors take layer = -1.  Storage follows the reference's policy
 * (Model::storage_dtype_for, model/model.cpp:959-986): norms, conv, dt_bias,
 * A_log, D, router and router bias are fp32; embeddings / lm_head fp16; every
 * other matrix is packed in the decoder's qkind (or fp16 when qkind is -1). */
enum {
    B200_T_EMBED = 0,        /* [vocab, hidden] fp16 */
    B200_T_FINAL_NORM = 1,   /* [hidden] fp32 */
    B200_T_LM_HEAD = 2,      /* [vocab, hidden] fp16 */
    B200_T_ROPE_INV_FREQ = 3,/* [head_dim/2] fp32 (only when rope_type >= 0) */
    B200_T_ATTN_NORM = 10,   /* [hidden] fp32: the norm before the mixer */
    B200_T_FFN_NORM = 11,    /* [hidden] fp32: the norm before the MoE */
    B200_T_MAMBA_IN = 20, B200_T_MAMBA_CONV_W = 21, B200_T_MAMBA_CONV_B = 22,
    B200_T_MAMBA_DT_BIAS = 23, B200_T_MAMBA_A_LOG = 24, B200_T_MAMBA_D = 25,
    B200_T_MAMBA_NORM = 26, B200_T_MAMBA_OUT = 27,
    B200_T_WQ = 30, B200_T_WK = 31, B200_T_WV = 32, B200_T_WO = 33,
    B200_T_ROUTER = 40, B200_T_ROUTER_BIAS = 41, B200_T_MOE_GATE = 42, B200_T_MOE_UP = 43,
    B200_T_MOE_DOWN = 44, B200_T_SH_GATE = 45, B200_T_SH_UP = 46, B200_T_SH_DOWN = 47
};

typedef struct b200_decoder b200_decoder;

/* layer_types[n_layers]: 0 = Mamba-2 layer, 1 = attention layer (ModelConfig::
 * layer_types, model/model.h).  rope_type: -1 none (NoPE), 0 interleaved, 1 neox.
 * attn_scale <= 0 selects 1/sqrt(head_dim).  max_ctx is the per-sequence KV
 * capacity (rounded up to whole pages of kv_page tokens). */
int b200_decoder_create(b200_decoder** out, int batch, int vocab, int hidden, int n_layers,
                        const int32_t* layer_types_host,
                        int n_heads, int n_kv_heads, int head_dim, int rope_type,
                        int mamba_heads, int mamba_d_head, int mamba_d_state, int mamba_d_conv,
                        int n_experts, int top_k, int expert_dim, int shared_dim,
                        int max_ctx, int kv_page, int qkind, float rms_eps,
                        float embedding_multiplier, float residual_multiplier, float attn_scale,
                        float logits_scaling);
int b200_decoder_destroy(b200_decoder* dec);
int b200_decoder_set_tensor(b200_decoder* dec, int layer, int tensor_id, const void* device_ptr);
/* Zero every sequence's Mamba state, conv window and KV length. */
int b200_decoder_reset(b200_decoder* dec);
/* fused = 0: one library op per reference op call, in the reference's order.
 * fused = 1: cross-op fusions (norm into the following projection's prologue,
 * residual add into the epilogue); returns B200_EUNSUPPORTED, leaving the mode
 * unchanged, when a matrix of the model cannot be cut into 16-byte-aligned row
 * tiles (the per-op mode has no such limit).
 * fused = 2 (batch 1 only): the Mamba and MoE phases of the token run inside one
 * persistent cooperative kernel per run of layers between attention layers (all CTAs
 * resident, weights streamed across phase boundaries, bounded grid barriers); attention
 * mixers and the lm_head use the fused = 1 kernels.  Needs every tensor set (it copies the
 * layer table to the device; b200_decoder_set_tensor afterwards drops back to fused = 0)
 * and widths that are multiples of 256; B200_EUNSUPPORTED otherwise.
 * use_graph = 1 captures the step once and replays it; the recording is dropped and made
 * again whenever one of the library's workspaces has been reallocated or released since. */
int b200_decoder_configure(b200_decoder* dec, int fused, int use_graph);
/* One token per sequence.  tokens_dev [batch] int32 in; next_dev [batch] int32 out
 * (greedy arg-max of the logits); both device pointers; no host synchronisation. */
int b200_decoder_step(b200_decoder* dec, const int32_t* tokens_dev, int32_t* next_dev);
/* The prompt: T tokens of every sequence at once (tokens_dev [batch, T] int32, sequence-
 * major) through the many-token kernels - what Generator::forward_prefill does with its
 * batched path (inference/generator.cpp:627-915), here including the Mamba layers.  The
 * sequences must be empty (after create or reset).  Afterwards the state is where T
 * calls of b200_decoder_step would have left it; next_dev (optional) receives the greedy
 * pick after the last prompt token, b200_decoder_logits its logits. */
int b200_decoder_prefill(b200_decoder* dec, const int32_t* tokens_dev, int T, int32_t* next_dev);
/* The same for prompts of different lengths (the batch-64 ragged prompt of a serving batch;
 * the reference would run them one after the other through Generator::prefill,
 * inference/generator.cpp:917-983): sequence b has lengths_host[b] tokens (1 .. max_ctx), the
 * sequences' tokens lie back to back in tokens_dev.  All token-wise work (projections, MoE,
 * norms) runs over the packed rows at once; the convolution window, the chunks of the SSD
 * scan, the causal attention and the KV pages never cross a sequence boundary.  Afterwards
 * every sequence stands where its own prefill would have left it, and b200_decoder_step
 * continues all of them (each at its own position); b200_decoder_position reports the longest. */
int b200_decoder_prefill_ragged(b200_decoder* dec, const int32_t* tokens_dev, const int32_t* lengths_host,
                                int32_t* next_dev);
/* Same through host buffers: H2D of the token ids, the step, D2H of the picks,
 * then a stream synchronise (what Generator::decode_step + ops::argmax_token do). */
int b200_decoder_step_host(b200_decoder* dec, const int32_t* tokens_host, int32_t* next_host);
/* Which position RoPE rotates by.  as_reference = 0 (default): the token's position in its
 * sequence.  as_reference = 1: what Generator::decode_step_logits does
 * (inference/generator.cpp:340-345): it uploads the position only while processing layer 0
 * and only if that layer is an attention layer, so on a hybrid model whose first layer is a
 * Mamba layer every token is rotated by the same never-refreshed word; a common rotation
 * leaves every q.k unchanged, so this mode applies no rotation on such models (and is the
 * default behaviour on all others).  Needed to reproduce the reference's own outputs on the
 * RoPE hybrid of the benchmark's first configuration; Granite-4.0-H itself has no RoPE. */
int b200_decoder_set_rope_refresh(b200_decoder* dec, int as_reference);
/* Diagnostic hook for the bounded grid barrier of the persistent step (fused = 2):
 * spin_limit > 0 replaces the iteration bound of its global-memory waits (0 restores the
 * default), skip_cta >= 0 makes that CTA leave at its first barrier without arriving (-1:
 * none).  With a CTA skipped the other CTAs' waits run out, the kernel returns and the step
 * reports B200_ECUDA through b200_decoder_step_host / b200_stream_status; the sequences'
 * state is then undefined until b200_decoder_reset. */
int b200_decoder_test_barrier(b200_decoder* dec, int spin_limit, int skip_cta);
/* Phase timers of the persistent step (the reference's phase timers, cuda/cuda_ops.h:315-319,
 * at the granularity of this kernel).  stamps_host == NULL arms (cta >= 0: the CTA that
 * records) or disarms (cta < 0) them; with a buffer of cap >= 4 * *n_phases entries it
 * synchronises and returns, per phase of the last step, four %globaltimer stamps in ns:
 * phase entered, activations staged, last tile done, barrier passed. */
int b200_decoder_phase_trace(b200_decoder* dec, int cta, uint64_t* stamps_host, int cap, int* n_phases);
/* Device pointer to the logits of the last step, [batch, vocab] fp32. */
int b200_decoder_logits(b200_decoder* dec, const float** logits_dev);
/* Tokens in each sequence's KV cache / state so far (all sequences advance together). */
int b200_decoder_position(b200_decoder* dec, int* position);
/* Kernel launches enqueued by one step in the current configuration. */
int b200_decoder_launches_per_step(b200_decoder* dec, int* launches);
/* Algorithmic bytes one step touches: every weight read once (K routed experts +
 * shared per token), Mamba state read+written, KV read for the current length. */
int b200_decoder_step_bytes(b200_decoder* dec, double* bytes);

/* ---- sampling tail on the device ----------------------------------------------------
 * The reference samples on the host after every token: Sampler::sample on a host copy of
 * the logits, or - its CUDA fast path, Generator::generate, inference/generator.cpp:1038-1056 -
 * penalties and top-K on the device, a copy of the K candidates to the host and
 * Sampler::sample_candidates there.  Here the generator state (core/rng.h: xoshiro256**
 * seeded by splitmix64), the token history and the pick stay in device memory. */
typedef struct b200_sampling {          /* SamplingConfig, inference/sampler.h:9-24 */
    float temperature, top_p, min_p, repetition_penalty, frequency_penalty, presence_penalty;
    int32_t top_k, repetition_window, no_repeat_ngram, greedy;
    uint64_t seed;
} b200_sampling;
/* The clamps of SamplingConfig::validate (inference/sampler.cpp:36-73), in place. */
int b200_sampling_validate(b200_sampling* cfg);
/* state_dev [streams, 4] uint64: stream i becomes Rng(seed + i) (core/rng.h:12-22). */
int b200_rng_seed(uint64_t seed, uint64_t* state_dev, int streams);
/* n values of Rng::uniform() (core/rng.h:39-41) from stream 0, which advances. */
int b200_rng_uniform(uint64_t* state_dev, float* out_dev, int n);
/* Sampler::sample_candidates (inference/sampler.cpp:194-266) for `rows` independent rows of
 * K <= 2048 candidates each (vals / ids [rows, K], any order): sort by value, softmax at the
 * temperature in double, min-p and top-p cuts, one uniform draw from row r's stream
 * (rng_state_dev + 4 r).  temperature <= 0 picks the largest.  next_dev [rows]. */
int b200_sample_candidates(const float* vals_dev, const int32_t* ids_dev, int K, int rows, const b200_sampling* cfg,
                           uint64_t* rng_state_dev, int32_t* next_dev);
/* Sampler::sample (inference/sampler.cpp:126-192) for `rows` rows of V logits, which are
 * modified in place as the reference's are: repetition / frequency / presence penalties over
 * the last repetition_window history tokens (0: all), the no-repeat n-gram ban, then greedy
 * pick, unfiltered softmax draw, or top-k / top-p / min-p draw.  hist_dev [rows, hist_stride]
 * int32 with hist_len_dev [rows] valid tokens each (oldest first; both NULL: no history);
 * hist_stride <= 8192 (Generator::HIST_MAX).  cfg is validated first. */
int b200_sample_logits(float* logits_dev, int V, int rows, const int32_t* hist_dev, int hist_stride,
                       const int32_t* hist_len_dev, const b200_sampling* cfg, uint64_t* rng_state_dev, int32_t* next_dev);
/* Makes b200_decoder_step / _prefill pick the next token by Sampler::sample instead of the
 * arg-max: the decoder keeps, per sequence, the history of fed tokens (ring of 8192) and a
 * generator stream Rng(cfg->seed + sequence), all on the device, so the step still runs
 * without host synchronisation and replays as one graph.  cfg == NULL returns to greedy.
 * History and streams start afresh here and at b200_decoder_reset. */
int b200_decoder_set_sampling(b200_decoder* dec, const b200_sampling* cfg);
/* Generator::score_tokens (inference/generator.cpp:1217-1294): the mean negative log-likelihood
 * of tokens[1..T) given their prefixes (position i predicts token i + 1; mask_host, optional,
 * [T] bytes: token i + 1 counts only if mask[i + 1] != 0), through the prompt kernels and a
 * chunked lm_head + cross-entropy (cuda/kernels.cu:1113-1200; sums in double as the CPU
 * function does, core/math_cpu.cpp:560-612).  Sequence 0 of an empty decoder (after create or
 * reset) is used and afterwards holds the T tokens.  T is cut to the decoder's context.  The
 * reference scores in windows of 512 tokens whose attention does not see earlier windows;
 * here every position sees its whole prefix (identical for T <= 513). */
int b200_decoder_score_tokens(b200_decoder* dec, const int32_t* tokens_host, int T, const uint8_t* mask_host,
                              double* mean_nll, int64_t* n_scored);

/* ---- quantisers on the device (reference host code: quant::quantize_q8_0 /
 * q4_0 / q4_1, quantization/quantize.cpp:20-246): kind 0 Q4_0, 1 Q4_1, 2 Q8_0; kind 3 =
 * Q4_K, this library's own single-pass quantiser; kind 4 = the Q4_0 layout filled by the
 * rule of the reference's GGUF writer (format/gguf_codec.cpp:408-460: scale from the signed
 * extreme, truncating codes).  n must be a multiple of the block size (256 for kind 3,
 * else 32); src 16-byte and dst 8-byte aligned.  Bit-identical to the CPU functions,
 * non-finite inputs included (the block becomes the zero block; under kind 4 a NaN that
 * is not the extreme gets code 0). */
int b200_quantize(const float* src, void* dst, int64_t n, int kind);

#ifdef __cplusplus
}
#endif
#endif /* B200STEP_H */
