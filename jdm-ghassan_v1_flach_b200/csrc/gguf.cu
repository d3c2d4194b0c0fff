// GGUF tensor ingest: the file is mapped, the tensor table parsed on the host, and each
// tensor is copied to the device - verbatim when the file already holds the wanted block
// layout, otherwise decoded to fp32 and converted / quantised by device kernels.
// Replaces GGUFReader::open / read_tensor_quant / read_tensor_raw and the per-parameter
// walk of load_model_from_gguf (format/gguf_codec.cpp:1445-1564) for the inference path.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <string>
#include <vector>

#include "quant.cuh"
#include "../../include/b200gguf.h"

extern "C" int b200_quantize(const float* src, void* dst, int64_t n, int kind);

namespace b200 {

struct GgufTensor {
    std::string name;
    std::vector<uint64_t> dims;      // as stored: innermost first
    uint32_t type = 0;
    uint64_t offset = 0, numel = 0, nbytes = 0;
};
struct GgufNumber {
    std::string key;
    double value;
};

// Elements per block and bytes per block of a GGML type; 0 elements = not handled here.
static void ggml_layout(uint32_t type, int& elems, int& bytes) {
    switch (type) {
        case B200_GGML_F32: elems = 1; bytes = 4; break;
        case B200_GGML_F16: elems = 1; bytes = 2; break;
        case B200_GGML_BF16: elems = 1; bytes = 2; break;
        case B200_GGML_Q4_0: elems = 32; bytes = 18; break;
        case B200_GGML_Q4_1: elems = 32; bytes = 20; break;
        case B200_GGML_Q8_0: elems = 32; bytes = 34; break;
        case B200_GGML_Q4_K: elems = 256; bytes = 144; break;
        default: elems = 0; bytes = 0; break;
    }
}
// storage kind <-> GGML type whose bytes are that kind's layout
static int kind_of_ggml(uint32_t type) {
    switch (type) {
        case B200_GGML_F32: return -2;
        case B200_GGML_F16: return -1;
        case B200_GGML_Q4_0: return 0;
        case B200_GGML_Q4_1: return 1;
        case B200_GGML_Q8_0: return 2;
        case B200_GGML_Q4_K: return 3;
        default: return -100;
    }
}
static uint64_t kind_bytes(int kind, uint64_t numel) {
    if (kind == -2) return numel * 4;
    if (kind == -1) return numel * 2;
    const int layout = kind == 4 ? 0 : kind;
    return numel / q_block_elems(layout) * q_block_bytes(layout);
}

// packed / half file bytes -> fp32 (exact values: d * q etc., as read_tensor_raw decodes them)
template <int KIND>
__global__ void gguf_decode_kernel(const uint8_t* __restrict__ src, float* __restrict__ dst, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        if (KIND >= 0) {
            dst[i] = q_value<KIND>(src, i);
        } else if (KIND == -1) {
            dst[i] = half_bits_to_float(reinterpret_cast<const uint16_t*>(src)[i]);
        } else {   // bf16
            dst[i] = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(src)[i] << 16);
        }
    }
}
__global__ void gguf_f32_to_f16_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = float_to_half_bits(src[i]);
}

}  // namespace b200

using namespace b200;

struct b200_gguf {
    int fd = -1;
    const uint8_t* map = nullptr;
    uint64_t size = 0, data_start = 0, alignment = 32;
    uint32_t version = 0;
    std::vector<GgufTensor> tensors;
    std::vector<GgufNumber> numbers;
};

namespace {
struct Cursor {
    const uint8_t* p;
    const uint8_t* end;
    bool ok = true;
    template <typename T>
    T pod() {
        T v{};
        if (!ok || (size_t)(end - p) < sizeof(T)) { ok = false; return v; }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = pod<uint64_t>();
        if (!ok || (uint64_t)(end - p) < n) { ok = false; return {}; }
        std::string s(reinterpret_cast<const char*>(p), (size_t)n);
        p += n;
        return s;
    }
    void skip(uint64_t n) {
        if (!ok || (uint64_t)(end - p) < n) { ok = false; return; }
        p += n;
    }
};
// GGUF metadata value types (format/gguf_codec.h:19-33)
enum { GT_U8 = 0, GT_I8, GT_U16, GT_I16, GT_U32, GT_I32, GT_F32, GT_BOOL, GT_STR, GT_ARR, GT_U64, GT_I64, GT_F64 };
int scalar_size(uint32_t t) {
    switch (t) {
        case GT_U8: case GT_I8: case GT_BOOL: return 1;
        case GT_U16: case GT_I16: return 2;
        case GT_U32: case GT_I32: case GT_F32: return 4;
        case GT_U64: case GT_I64: case GT_F64: return 8;
        default: return 0;
    }
}
bool read_value(Cursor& c, uint32_t type, double* number) {
    switch (type) {
        case GT_U8: *number = c.pod<uint8_t>(); return true;
        case GT_I8: *number = c.pod<int8_t>(); return true;
        case GT_U16: *number = c.pod<uint16_t>(); return true;
        case GT_I16: *number = c.pod<int16_t>(); return true;
        case GT_U32: *number = c.pod<uint32_t>(); return true;
        case GT_I32: *number = c.pod<int32_t>(); return true;
        case GT_F32: *number = c.pod<float>(); return true;
        case GT_BOOL: *number = c.pod<uint8_t>() ? 1.0 : 0.0; return true;
        case GT_U64: *number = (double)c.pod<uint64_t>(); return true;
        case GT_I64: *number = (double)c.pod<int64_t>(); return true;
        case GT_F64: *number = c.pod<double>(); return true;
        case GT_STR: c.str(); return false;
        case GT_ARR: {
            const uint32_t et = c.pod<uint32_t>();
            const uint64_t n = c.pod<uint64_t>();
            if (et == GT_STR) {
                for (uint64_t i = 0; i < n && c.ok; ++i) c.str();
            } else if (et == GT_ARR || scalar_size(et) == 0) {
                c.ok = false;        // nested arrays are not part of the format
            } else {
                c.skip(n * (uint64_t)scalar_size(et));
            }
            return false;
        }
        default: c.ok = false; return false;
    }
}
}  // namespace

extern "C" {

int b200_gguf_open(const char* path, b200_gguf** out) {
    B200_REQUIRE(path && out, "gguf_open: null pointer");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(B200_EINVAL, "gguf_open: cannot open %s", path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) {
        close(fd);
        return fail(B200_EINVAL, "gguf_open: %s is not a GGUF file (too short)", path);
    }
    void* map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) {
        close(fd);
        return fail(B200_ENOMEM, "gguf_open: mmap of %s failed", path);
    }
    b200_gguf* g = new b200_gguf();
    g->fd = fd;
    g->map = static_cast<const uint8_t*>(map);
    g->size = (uint64_t)st.st_size;
    Cursor c{g->map, g->map + g->size};
    const uint32_t magic = c.pod<uint32_t>();
    g->version = c.pod<uint32_t>();
    auto bail = [&](const char* why) {
        b200_gguf_close(g);
        return fail(B200_EINVAL, "gguf_open: %s: %s", path, why);
    };
    if (magic != 0x46554747u) return bail("bad magic");
    if (g->version != 2 && g->version != 3) return bail("unsupported GGUF version");
    const uint64_t n_tensors = c.pod<uint64_t>(), n_kv = c.pod<uint64_t>();
    if (!c.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) return bail("implausible header counts");
    for (uint64_t i = 0; i < n_kv; ++i) {
        const std::string key = c.str();
        const uint32_t type = c.pod<uint32_t>();
        double num = 0.0;
        const bool numeric = read_value(c, type, &num);
        if (!c.ok) return bail("truncated or malformed metadata");
        if (numeric) {
            g->numbers.push_back({key, num});
            if (key == "general.alignment") {
                // a power of two of at most 1 MiB, as every writer produces; anything else is a damaged file
                const uint64_t a = num >= 1.0 && num <= 1048576.0 ? (uint64_t)num : 0;
                if (a == 0 || (a & (a - 1)) != 0) return bail("implausible general.alignment");
                g->alignment = a;
            }
        }
    }
    g->tensors.resize((size_t)n_tensors);
    for (GgufTensor& t : g->tensors) {
        t.name = c.str();
        const uint32_t nd = c.pod<uint32_t>();
        if (!c.ok || nd > 4) return bail("tensor with more than four dimensions");
        t.numel = 1;
        for (uint32_t k = 0; k < nd; ++k) {
            const uint64_t dim = c.pod<uint64_t>();
            // (a product beyond 2^40 elements cannot lie inside a file; refusing it here also keeps
            // the multiplication from wrapping)
            if (dim == 0 || dim > ((uint64_t)1 << 40) || t.numel > ((uint64_t)1 << 40) / dim) return bail("implausible tensor shape");
            t.dims.push_back(dim);
            t.numel *= dim;
        }
        t.type = c.pod<uint32_t>();
        t.offset = c.pod<uint64_t>();
        int be, bb;
        ggml_layout(t.type, be, bb);
        t.nbytes = be ? (t.numel + be - 1) / be * (uint64_t)bb : 0;
    }
    if (!c.ok) return bail("truncated tensor table");
    const uint64_t here = (uint64_t)(c.p - g->map);
    g->data_start = (here + g->alignment - 1) / g->alignment * g->alignment;
    for (const GgufTensor& t : g->tensors) {
        // same bounds the reference checks (format/gguf_codec.cpp:1476-1479)
        if (g->data_start > g->size || t.offset > g->size - g->data_start ||
            t.nbytes > g->size - g->data_start - t.offset) {
            b200_gguf_close(g);
            return fail(B200_EINVAL, "gguf_open: %s: tensor %s lies outside the file", path, t.name.c_str());
        }
    }
    *out = g;
    return B200_OK;
}

int b200_gguf_close(b200_gguf* g) {
    if (!g) return B200_OK;
    if (g->map) munmap(const_cast<uint8_t*>(g->map), (size_t)g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
    return B200_OK;
}

int b200_gguf_tensor_count(b200_gguf* g, int* count) {
    B200_REQUIRE(g && count, "gguf_tensor_count: null pointer");
    *count = (int)g->tensors.size();
    return B200_OK;
}

int b200_gguf_tensor_info(b200_gguf* g, int index, char* name, int name_cap, int64_t* dims, int* n_dims,
                          int* ggml_type, uint64_t* nbytes) {
    B200_REQUIRE(g && index >= 0 && index < (int)g->tensors.size(), "gguf_tensor_info: index out of range");
    const GgufTensor& t = g->tensors[(size_t)index];
    if (name && name_cap > 0) snprintf(name, (size_t)name_cap, "%s", t.name.c_str());
    if (dims) {
        for (int k = 0; k < 4; ++k) dims[k] = 1;
        const int nd = (int)t.dims.size();
        for (int k = 0; k < nd; ++k) dims[k] = (int64_t)t.dims[(size_t)(nd - 1 - k)];     // outermost first
    }
    if (n_dims) *n_dims = (int)t.dims.size();
    if (ggml_type) *ggml_type = (int)t.type;
    if (nbytes) *nbytes = t.nbytes;
    return B200_OK;
}

int b200_gguf_tensor_data(b200_gguf* g, int index, const void** host_ptr) {
    B200_REQUIRE(g && host_ptr && index >= 0 && index < (int)g->tensors.size(), "gguf_tensor_data: bad arguments");
    *host_ptr = g->map + g->data_start + g->tensors[(size_t)index].offset;
    return B200_OK;
}

int b200_gguf_find_tensor(b200_gguf* g, const char* name, int* index) {
    B200_REQUIRE(g && name && index, "gguf_find_tensor: null pointer");
    *index = -1;
    for (size_t i = 0; i < g->tensors.size(); ++i)
        if (g->tensors[i].name == name) { *index = (int)i; break; }
    return B200_OK;
}

int b200_gguf_metadata_number(b200_gguf* g, const char* key, double* value) {
    B200_REQUIRE(g && key && value, "gguf_metadata_number: null pointer");
    for (const GgufNumber& n : g->numbers)
        if (n.key == key) { *value = n.value; return B200_OK; }
    return fail(B200_EINVAL, "gguf_metadata_number: no numeric key %s", key);
}

int b200_gguf_storage_kind(const char* param_name, int quant_kind, int* kind) {
    B200_REQUIRE(param_name && kind, "gguf_storage_kind: null pointer");
    B200_REQUIRE(quant_kind >= -1 && quant_kind <= 4, "gguf_storage_kind: unknown quant_kind %d", quant_kind);
    const std::string n(param_name);
    auto has = [&](const char* s) { return n.find(s) != std::string::npos; };
    if (n == "tok_embeddings" || n == "lm_head") { *kind = -1; return B200_OK; }
    const bool fragile = has("lora_") || has("moe_router") || has("mamba.conv1d") || has("mamba.dt_bias") ||
                         has("mamba.A_log") || has("mamba.D") || has("norm") || has("bias") || has(".bq") ||
                         has(".bk") || has(".bv");
    *kind = fragile ? -2 : quant_kind;
    return B200_OK;
}

int b200_gguf_tensor_bytes(b200_gguf* g, int index, int kind, uint64_t* bytes) {
    B200_REQUIRE(g && bytes && index >= 0 && index < (int)g->tensors.size(), "gguf_tensor_bytes: bad arguments");
    B200_REQUIRE(kind >= -2 && kind <= 4, "gguf_tensor_bytes: unknown kind %d", kind);
    const GgufTensor& t = g->tensors[(size_t)index];
    if (kind >= 0) B200_REQUIRE(t.numel % q_block_elems(kind == 4 ? 0 : kind) == 0, "gguf_tensor_bytes: %s is not a whole number of blocks", t.name.c_str());
    *bytes = kind_bytes(kind, t.numel);
    return B200_OK;
}

int b200_gguf_load_tensor(b200_gguf* g, int index, int kind, void* device_dst, uint64_t dst_bytes) {
    B200_REQUIRE(g && device_dst && index >= 0 && index < (int)g->tensors.size(), "gguf_load_tensor: bad arguments");
    B200_REQUIRE(kind >= -2 && kind <= 4, "gguf_load_tensor: unknown kind %d", kind);
    const GgufTensor& t = g->tensors[(size_t)index];
    int be, bb;
    ggml_layout(t.type, be, bb);
    if (be == 0) return fail(B200_EUNSUPPORTED, "gguf_load_tensor: %s has GGML type %u, which this loader does not decode", t.name.c_str(), t.type);
    if (kind >= 0) B200_REQUIRE(t.numel % q_block_elems(kind == 4 ? 0 : kind) == 0, "gguf_load_tensor: %s is not a whole number of blocks of the target kind", t.name.c_str());
    B200_REQUIRE(t.numel % be == 0, "gguf_load_tensor: %s is not a whole number of blocks in the file", t.name.c_str());
    const uint64_t need = kind_bytes(kind, t.numel);
    B200_REQUIRE(dst_bytes >= need, "gguf_load_tensor: destination of %llu bytes, %llu needed", (unsigned long long)dst_bytes, (unsigned long long)need);
    const uint8_t* src = g->map + g->data_start + t.offset;
    cudaStream_t st = stream();
    if (kind_of_ggml(t.type) == kind) {
        // the file already stores this exact layout: the bytes go as they are
        B200_CUDA(cudaMemcpyAsync(device_dst, src, (size_t)t.nbytes, cudaMemcpyHostToDevice, st));
        B200_CUDA(cudaStreamSynchronize(st));
        return B200_OK;
    }
    // decode to fp32 on the device, then convert / quantise
    uint8_t* raw = nullptr;
    float* f32 = nullptr;
    const int64_t n = (int64_t)t.numel;
    auto cleanup = [&]() {
        if (raw) cudaFree(raw);
        if (f32 && static_cast<void*>(f32) != device_dst) cudaFree(f32);
    };
    cudaError_t e = cudaMalloc(&raw, (size_t)t.nbytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(raw, src, (size_t)t.nbytes, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) {
        if (kind == -2) f32 = static_cast<float*>(device_dst);
        else e = cudaMalloc(&f32, (size_t)n * 4);
    }
    if (e != cudaSuccess) {
        cleanup();
        return cuda_status(e, "gguf_load_tensor: staging");
    }
    const unsigned grid = (unsigned)std::min<int64_t>(ceil_div64(n, 256), (int64_t)num_sms() * 16);
    switch (t.type) {
        case B200_GGML_F32: e = cudaMemcpyAsync(f32, raw, (size_t)n * 4, cudaMemcpyDeviceToDevice, st); break;
        case B200_GGML_F16: gguf_decode_kernel<-1><<<grid, 256, 0, st>>>(raw, f32, n); break;
        case B200_GGML_BF16: gguf_decode_kernel<-3><<<grid, 256, 0, st>>>(raw, f32, n); break;
        case B200_GGML_Q4_0: gguf_decode_kernel<0><<<grid, 256, 0, st>>>(raw, f32, n); break;
        case B200_GGML_Q4_1: gguf_decode_kernel<1><<<grid, 256, 0, st>>>(raw, f32, n); break;
        case B200_GGML_Q8_0: gguf_decode_kernel<2><<<grid, 256, 0, st>>>(raw, f32, n); break;
        default: gguf_decode_kernel<3><<<grid, 256, 0, st>>>(raw, f32, n); break;
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    int rc = e == cudaSuccess ? B200_OK : cuda_status(e, "gguf_load_tensor: decode");
    ++g_kernel_launches;
    if (!rc && kind == -1) {
        gguf_f32_to_f16_kernel<<<grid, 256, 0, st>>>(f32, static_cast<uint16_t*>(device_dst), n);
        e = cudaGetLastError();
        if (e != cudaSuccess) rc = cuda_status(e, "gguf_load_tensor: fp16 conversion");
        ++g_kernel_launches;
    } else if (!rc && kind >= 0) {
        rc = b200_quantize(f32, device_dst, n, kind);
    }
    e = cudaStreamSynchronize(st);
    if (!rc && e != cudaSuccess) rc = cuda_status(e, "gguf_load_tensor: synchronize");
    cleanup();
    return rc;
}

}  // extern "C"
