/* b200gguf - GGUF tensor ingest straight into device memory.
 *
 * The reference engine loads a GGUF checkpoint tensor by tensor through host
 * staging (GGUFReader::read_tensor_quant, format/gguf_codec.cpp:1445-1500: a verbatim
 * block copy when the file already holds the wanted layout, else decode to fp32 and
 * quantise on the CPU; load_model_from_gguf, :1507-1564, walks the model's parameters).
 * Here the file is mapped, the tensor table parsed once, and each tensor goes to the
 * caller's device buffer in the storage kind asked for: packed blocks are copied as
 * they are, anything else is decoded and re-quantised by device kernels (the
 * load-time quantisation the reference does on the host).
 *
 * Storage kinds ("kind" below): -2 fp32, -1 fp16, 0 Q4_0, 1 Q4_1, 2 Q8_0, 3 Q4_K
 * (the qkind values of b200ops.h), 4 = Q4_0 filled by the GGUF writer's rule.
 */
#ifndef B200GGUF_H
#define B200GGUF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200_gguf b200_gguf;

/* GGML type ids as stored in the file (format/gguf_codec.h:35-50). */
enum {
    B200_GGML_F32 = 0, B200_GGML_F16 = 1, B200_GGML_Q4_0 = 2, B200_GGML_Q4_1 = 3, B200_GGML_Q8_0 = 8,
    B200_GGML_Q4_K = 12, B200_GGML_BF16 = 30
};

/* Maps the file read-only and parses header, metadata and tensor table (GGUF version 2
 * or 3; GGUFReader::open, format/gguf_codec.cpp).  No device work. */
int b200_gguf_open(const char* path, b200_gguf** out);
int b200_gguf_close(b200_gguf* g);
int b200_gguf_tensor_count(b200_gguf* g, int* count);
/* name_cap bytes for the name (NUL-terminated, truncated if longer); dims[4] outermost
 * first (the file stores them innermost first), unused entries 1. */
int b200_gguf_tensor_info(b200_gguf* g, int index, char* name, int name_cap, int64_t* dims, int* n_dims,
                          int* ggml_type, uint64_t* nbytes);
/* Host pointer to the tensor's bytes inside the mapping (valid until b200_gguf_close). */
int b200_gguf_tensor_data(b200_gguf* g, int index, const void** host_ptr);
/* Index of the tensor with exactly this name, -1 in *index if the file has none. */
int b200_gguf_find_tensor(b200_gguf* g, const char* name, int* index);
/* Numeric metadata value as a double (unsigned / signed integers, floats, bools);
 * B200_EINVAL when the key is absent or not numeric. */
int b200_gguf_metadata_number(b200_gguf* g, const char* key, double* value);
/* The storage kind the engine keeps a parameter in when it runs with packed weights of
 * quant_kind (Model::storage_dtype_for, model/model.cpp:959-986): norms, conv1d, dt_bias,
 * A_log, D, router, biases fp32 (-2); tok_embeddings / lm_head fp16 (-1); every other
 * matrix quant_kind. */
int b200_gguf_storage_kind(const char* param_name, int quant_kind, int* kind);
/* Bytes tensor `index` occupies in storage kind `kind`. */
int b200_gguf_tensor_bytes(b200_gguf* g, int index, int kind, uint64_t* bytes);
/* Tensor `index` into device_dst (>= the bytes above) in storage kind `kind`, enqueued on
 * the library's stream: a host-to-device copy of the file's bytes when the file already
 * stores that layout (GGUFReader::read_tensor_quant's fast path), otherwise decode to
 * fp32 and convert / quantise on the device (its slow path; bit-identical to the host
 * quantisers).  Synchronises before returning (the staging buffers are freed). */
int b200_gguf_load_tensor(b200_gguf* g, int index, int kind, void* device_dst, uint64_t dst_bytes);

#ifdef __cplusplus
}
#endif
#endif /* B200GGUF_H */
