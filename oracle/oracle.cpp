// CPU oracle for the quantized hybrid-layer forward step (Mamba-2 + GQA + MoE).
//
// TEST INFRASTRUCTURE ONLY.  This file restates, in plain scalar C++, the
// arithmetic of the reference engine's CPU path so that the CUDA library can be
// checked against it.  Nothing in the product path may call it: the CUDA library
// has no CPU fallback.  Only the test-suite, the smoke check and the CPU-baseline
// leg of the benchmark load the shared object built from this file.
//
// Every function names the reference file:line whose arithmetic it follows.
// Compile with -ffp-contract=off: the reference's default build targets baseline
// x86-64 (no FMA contraction), and the bit-exact checks (dequantised weights,
// router top-k) rely on separate multiply and add roundings.
//
// Parity status.  The reference ships no golden vectors for this path; the oracle
// is pinned by running the reference's own CPU objects (compiled from the
// reference sources by oracle/Makefile into oracle/_ref/) on the same seeded
// inputs (tests/test_oracle_vs_ref.py) and by the fixtures under tests/golden/
// generated from those objects.  Q4_K is absent from the reference (its codec only
// knows the GGML type id), so the Q4_K block arithmetic below restates the public
// GGML block layout (ggml, unpinned - the reference vendors no copy): for Q4_K
// "parity unpinned".
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

typedef uint8_t u8;
typedef int8_t i8;
typedef uint16_t u16;
typedef int32_t i32;
typedef int64_t i64;
typedef uint64_t u64;

#define ORA_API extern "C" __attribute__((visibility("default")))

// ----------------------------------------------------------------------------
// fp16 <-> fp32, round-to-nearest-even.  Follows core/dtype.h:61-112.
// ----------------------------------------------------------------------------
static inline u16 f32_to_f16_bits(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t e8 = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (e8 == 0xFFu) return (u16)(sign | 0x7C00u | (man ? 0x200u : 0u));
    const int e = (int)e8 - 127 + 15;
    if (e >= 31) return (u16)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (u16)sign;
        man |= 0x800000u;
        const uint32_t sh = (uint32_t)(14 - e);
        uint32_t sub = man >> sh;
        const uint32_t halfway = 1u << (sh - 1);
        const uint32_t rest = man & ((1u << sh) - 1u);
        if (rest > halfway || (rest == halfway && (sub & 1u))) ++sub;
        return (u16)(sign | sub);
    }
    u16 h = (u16)(sign | ((uint32_t)e << 10) | (man >> 13));
    const uint32_t tail = man & 0x1FFFu;
    if (tail > 0x1000u || (tail == 0x1000u && (h & 1u))) ++h;
    return h;
}

static inline float f16_bits_to_f32(u16 h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e5 = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (e5 == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int shift = 0;
            while ((man & 0x400u) == 0) { man <<= 1; ++shift; }
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
        }
    } else if (e5 == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((e5 - 15 + 127) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

ORA_API void ora_f32_to_f16(const float* src, u16* dst, i64 n) {
    for (i64 i = 0; i < n; ++i) dst[i] = f32_to_f16_bits(src[i]);
}
ORA_API void ora_f16_to_f32(const u16* src, float* dst, i64 n) {
    for (i64 i = 0; i < n; ++i) dst[i] = f16_bits_to_f32(src[i]);
}

static inline u16 rd16(const u8* p) { return (u16)(p[0] | (p[1] << 8)); }

// ----------------------------------------------------------------------------
// Packed block formats.  kind 0 = Q4_0 (18 B / 32), 1 = Q4_1 (20 B / 32),
// 2 = Q8_0 (34 B / 32) follow core/dtype.h:35-53; kind 3 = Q4_K (144 B / 256:
// f16 d, f16 dmin, 12 B of packed 6-bit scales/mins, 128 B of nibbles) follows
// the public GGML layout.
// ----------------------------------------------------------------------------
static inline int kind_block_elems(int kind) { return kind == 3 ? 256 : 32; }
static inline int kind_block_bytes(int kind) {
    return kind == 0 ? 18 : kind == 1 ? 20 : kind == 2 ? 34 : 144;
}

ORA_API i64 ora_packed_bytes(int kind, i64 n) {
    const int be = kind_block_elems(kind);
    return ((n + be - 1) / be) * (i64)kind_block_bytes(kind);
}

// 6-bit (scale, min) pair number j (0..7) of a Q4_K super-block.
static inline void q4k_scale_min(int j, const u8* sc, int* s, int* m) {
    if (j < 4) {
        *s = sc[j] & 63;
        *m = sc[j + 4] & 63;
    } else {
        *s = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4);
        *m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
    }
}

// One dequantised weight, fp32, before the fp16 rounding of the inference path.
// kinds 0..2: core/ops.cpp:313-334 (same arithmetic as quantization/quantize.cpp
// dequantize_*): separate multiply and add.
static inline float dequant_one(const u8* packed, int kind, i64 i) {
    if (kind == 3) {
        const u8* blk = packed + (i >> 8) * 144;
        const int r = (int)(i & 255);
        const int grp = r >> 6;          // 64 weights share 32 nibble bytes
        const int hi = (r >> 5) & 1;     // second half of the group = high nibbles
        const int l = r & 31;
        int s, m;
        q4k_scale_min(2 * grp + hi, blk + 4, &s, &m);
        const float d = f16_bits_to_f32(rd16(blk));
        const float dmin = f16_bits_to_f32(rd16(blk + 2));
        const u8 byte = blk[16 + 32 * grp + l];
        const int q = hi ? (byte >> 4) : (byte & 0x0F);
        const float d1 = d * (float)s;
        const float m1 = dmin * (float)m;
        return d1 * (float)q - m1;
    }
    const i64 b = i >> 5;
    const int j = (int)(i & 31);
    if (kind == 0) {
        const u8* blk = packed + b * 18;
        const float d = f16_bits_to_f32(rd16(blk));
        const u8 byte = blk[2 + (j & 15)];
        const int q = (j < 16) ? (byte & 0x0F) : (byte >> 4);
        return (float)(q - 8) * d;
    }
    if (kind == 1) {
        const u8* blk = packed + b * 20;
        const float d = f16_bits_to_f32(rd16(blk));
        const float mn = f16_bits_to_f32(rd16(blk + 2));
        const u8 byte = blk[4 + (j & 15)];
        const int q = (j < 16) ? (byte & 0x0F) : (byte >> 4);
        const float t = (float)q * d;
        return t + mn;
    }
    const u8* blk = packed + b * 34;
    const float d = f16_bits_to_f32(rd16(blk));
    return (float)((const i8*)(blk + 2))[j] * d;
}

// The weight value a linear layer multiplies with.  Default: rounded through fp16,
// as the reference's CPU inference path does (core/ops.cpp:335,392).  With rounding
// switched off it is the exact dequantised value, which is what the reference's
// fused CUDA kernel (cuda/kernels.cu:549-598) and this repository's kernels use;
// the two differ by a 2^-12 relative perturbation per weight.
static bool g_round_weights = true;
ORA_API void ora_set_weight_rounding(int on) { g_round_weights = on != 0; }
static inline float weight_value(const u8* packed, int kind, i64 i) {
    const float v = dequant_one(packed, kind, i);
    return g_round_weights ? f16_bits_to_f32(f32_to_f16_bits(v)) : v;
}

// Packed -> fp16, the form the reference's CPU inference path consumes
// (ops::quant_materialize, core/ops.cpp:304-338).
ORA_API void ora_dequantize(const void* packed, u16* dst, i64 n, int kind) {
    const u8* p = (const u8*)packed;
#pragma omp parallel for schedule(static) if (n > 65536)
    for (i64 i = 0; i < n; ++i) dst[i] = f32_to_f16_bits(dequant_one(p, kind, i));
}

// Packed -> fp32 without the fp16 rounding (quantization/quantize.cpp:76-95,
// 158-185, 248-277).
ORA_API void ora_dequantize_f32(const void* packed, float* dst, i64 n, int kind) {
    const u8* p = (const u8*)packed;
#pragma omp parallel for schedule(static) if (n > 65536)
    for (i64 i = 0; i < n; ++i) dst[i] = dequant_one(p, kind, i);
}

// ----------------------------------------------------------------------------
// Quantizers.  Q8_0 / Q4_0 / Q4_1 follow quantization/quantize.cpp:20-246 for
// whole blocks (n must be a multiple of 32 here; the ragged tail of the reference
// is not on the inference path).  Rounding is lround (half away from zero).
// ----------------------------------------------------------------------------
static inline void wr16(u8* p, u16 v) { p[0] = (u8)(v & 0xFF); p[1] = (u8)(v >> 8); }

static inline int iclamp(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

ORA_API int ora_quantize(const float* src, void* dst, i64 n, int kind);

static void quant_block_q8_0(const float* x, u8* out) {
    float amax = 0.0f;
    bool bad = false;
    for (int i = 0; i < 32; ++i) {
        if (!std::isfinite(x[i])) { bad = true; break; }
        amax = std::max(amax, std::fabs(x[i]));
    }
    if (bad) { wr16(out, f32_to_f16_bits(0.0f)); std::memset(out + 2, 0, 32); return; }
    const float scale = amax / 127.0f;
    const float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
    wr16(out, f32_to_f16_bits(scale));
    for (int i = 0; i < 32; ++i)
        ((i8*)(out + 2))[i] = (i8)iclamp((int)std::lround(x[i] * inv), -127, 127);
}

static void quant_block_q4_0(const float* x, u8* out) {
    float amax = 0.0f;
    bool bad = false;
    for (int i = 0; i < 32; ++i) {
        if (!std::isfinite(x[i])) { bad = true; break; }
        amax = std::max(amax, std::fabs(x[i]));
    }
    if (bad) { wr16(out, f32_to_f16_bits(0.0f)); std::memset(out + 2, 0x88, 16); return; }
    const float scale = amax / 8.0f;
    const float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
    wr16(out, f32_to_f16_bits(scale));
    for (int j = 0; j < 16; ++j) {
        const int lo = iclamp((int)std::lround(x[j] * inv), -8, 7) + 8;
        const int hi = iclamp((int)std::lround(x[j + 16] * inv), -8, 7) + 8;
        out[2 + j] = (u8)((hi << 4) | lo);
    }
}

// Q4_0 as the GGUF writer packs it (format/gguf_codec.cpp:408-460, GGML's
// quantize_row_q4_0_ref): the scale follows the SIGNED extreme, d = vmax / -8 with vmax
// the first element of largest magnitude; codes min(15, (int)(x / d + 8.5)), truncated.
// A block that is all zero or holds a non-finite value becomes the zero block.
static void quant_block_q4_0_ggml(const float* x, u8* out) {
    float amax = 0.0f, vmax = 0.0f;
    for (int i = 0; i < 32; ++i) {
        const float a = std::fabs(x[i]);
        if (a > amax) { amax = a; vmax = x[i]; }
    }
    const bool bad = !std::isfinite(amax) || amax == 0.0f;
    if (bad) { wr16(out, f32_to_f16_bits(0.0f)); std::memset(out + 2, 0x88, 16); return; }
    const float d = vmax / -8.0f;
    const float id = 1.0f / d;
    wr16(out, f32_to_f16_bits(d));
    for (int j = 0; j < 16; ++j) {
        // a NaN element never wins `a > amax`; its code is what the reference's float -> int
        // conversion yields on x86 (INT_MIN) after the clamp: 0
        const float f0 = x[j] * id + 8.5f, f1 = x[j + 16] * id + 8.5f;
        const int lo = std::isnan(f0) ? 0 : iclamp((int)f0, 0, 15);
        const int hi = std::isnan(f1) ? 0 : iclamp((int)f1, 0, 15);
        out[2 + j] = (u8)((hi << 4) | lo);
    }
}

static void quant_block_q4_1(const float* x, u8* out) {
    for (int i = 0; i < 32; ++i)
        if (!std::isfinite(x[i])) { std::memset(out, 0, 20); return; }
    float mn = x[0], mx = x[0];
    for (int i = 1; i < 32; ++i) { mn = std::min(mn, x[i]); mx = std::max(mx, x[i]); }
    const float scale = (mx - mn) / 15.0f;
    const float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
    wr16(out, f32_to_f16_bits(scale));
    wr16(out + 2, f32_to_f16_bits(mn));
    for (int j = 0; j < 16; ++j) {
        const int lo = iclamp((int)std::lround((x[j] - mn) * inv), 0, 15);
        const int hi = iclamp((int)std::lround((x[j + 16] - mn) * inv), 0, 15);
        out[4 + j] = (u8)((hi << 4) | lo);
    }
}

// Q4_K quantizer (this project's own; the reference has none).  One pass, no
// iterative scale search: per 32-weight sub-block take lo = min(x, 0) and
// scale = (max - lo) / 15; the super-block scales are max(scale)/63 and
// max(-lo)/63 stored as fp16; 6-bit codes by round-half-up; nibbles from the
// fp16-rounded super-block scales so that decode(encode(x)) is self-consistent.
// Every step is a single fp32 operation so the CUDA quantizer can be bit-exact.
static inline int round_half_up(float v) { return (int)std::floor(v + 0.5f); }

static void quant_block_q4_k(const float* x, u8* out) {
    float sc[8], mnv[8];
    float max_sc = 0.0f, max_mn = 0.0f;
    bool bad = false;
    for (int i = 0; i < 256; ++i)
        if (!std::isfinite(x[i])) { bad = true; break; }
    if (bad) { std::memset(out, 0, 144); return; }
    for (int s = 0; s < 8; ++s) {
        float lo = 0.0f, hi = x[32 * s];
        for (int i = 0; i < 32; ++i) {
            lo = std::min(lo, x[32 * s + i]);
            hi = std::max(hi, x[32 * s + i]);
        }
        if (hi < lo) hi = lo;
        sc[s] = (hi - lo) / 15.0f;
        mnv[s] = -lo;
        max_sc = std::max(max_sc, sc[s]);
        max_mn = std::max(max_mn, mnv[s]);
    }
    const float inv_sc = max_sc > 0.0f ? 63.0f / max_sc : 0.0f;
    const float inv_mn = max_mn > 0.0f ? 63.0f / max_mn : 0.0f;
    int ls[8], lm[8];
    for (int s = 0; s < 8; ++s) {
        ls[s] = iclamp(round_half_up(inv_sc * sc[s]), 0, 63);
        lm[s] = iclamp(round_half_up(inv_mn * mnv[s]), 0, 63);
    }
    const u16 d16 = f32_to_f16_bits(max_sc / 63.0f);
    const u16 m16 = f32_to_f16_bits(max_mn / 63.0f);
    wr16(out, d16);
    wr16(out + 2, m16);
    u8* scales = out + 4;
    std::memset(scales, 0, 12);
    for (int j = 0; j < 8; ++j) {
        if (j < 4) {
            scales[j] = (u8)ls[j];
            scales[j + 4] = (u8)lm[j];
        } else {
            scales[j + 4] = (u8)((ls[j] & 0x0F) | ((lm[j] & 0x0F) << 4));
            scales[j - 4] |= (u8)((ls[j] >> 4) << 6);
            scales[j] |= (u8)((lm[j] >> 4) << 6);
        }
    }
    const float d = f16_bits_to_f32(d16);
    const float dmin = f16_bits_to_f32(m16);
    u8 q[256];
    for (int s = 0; s < 8; ++s) {
        const float dd = d * (float)ls[s];
        const float dm = dmin * (float)lm[s];
        for (int i = 0; i < 32; ++i) {
            int v = 0;
            if (dd > 0.0f) v = iclamp(round_half_up((x[32 * s + i] + dm) / dd), 0, 15);
            q[32 * s + i] = (u8)v;
        }
    }
    u8* qs = out + 16;
    for (int g = 0; g < 4; ++g)
        for (int l = 0; l < 32; ++l)
            qs[32 * g + l] = (u8)(q[64 * g + l] | (q[64 * g + 32 + l] << 4));
}

// kind 4: the Q4_0 layout (kind 0) filled by the GGUF writer's rule.
ORA_API int ora_quantize(const float* src, void* dst, i64 n, int kind) {
    const int layout = kind == 4 ? 0 : kind;
    const int be = kind_block_elems(layout);
    if (n < 0 || n % be != 0) return -1;
    const int bb = kind_block_bytes(layout);
    u8* out = (u8*)dst;
    const i64 nb = n / be;
#pragma omp parallel for schedule(static) if (nb > 1024)
    for (i64 b = 0; b < nb; ++b) {
        const float* x = src + b * be;
        u8* o = out + b * bb;
        if (kind == 0) quant_block_q4_0(x, o);
        else if (kind == 4) quant_block_q4_0_ggml(x, o);
        else if (kind == 1) quant_block_q4_1(x, o);
        else if (kind == 2) quant_block_q8_0(x, o);
        else quant_block_q4_k(x, o);
    }
    return 0;
}

// ----------------------------------------------------------------------------
// Linear layers: y[M,N] = x[M,K] . W^T, W row-major [N,K].
// ----------------------------------------------------------------------------

// Packed weights: the row is dequantised to fp16 and the dot product runs in
// fp32 in k order (ops::linear_forward_q4 CPU mirror, core/ops.cpp:360-401).
ORA_API int ora_linear_q4(const float* x, const void* w, float* y, int M, int K, int N, int kind) {
    if (M <= 0 || N <= 0) return 0;
    const int be = kind_block_elems(kind);
    if (K % be != 0) return -1;
    const u8* p = (const u8*)w;
    const i64 row_bytes = (i64)(K / be) * kind_block_bytes(kind);
#pragma omp parallel for schedule(static) if ((i64)N * K > 65536)
    for (int n = 0; n < N; ++n) {
        std::vector<float> row((size_t)K);
        const u8* wr = p + (i64)n * row_bytes;
        for (int k = 0; k < K; ++k) row[k] = weight_value(wr, kind, k);
        for (int m = 0; m < M; ++m) {
            const float* xa = x + (size_t)m * K;
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += xa[k] * row[k];
            y[(size_t)m * N + n] = acc;
        }
    }
    return 0;
}

// The same product without the fp16 rounding of each dequantised weight: what the
// reference's fused CUDA kernel computes (q4_val keeps fp32, cuda/kernels.cu:549-598).
// The tensor-core kernels are held to this variant tightly and to the rounded CPU
// variant above within the stated activation tolerance.
ORA_API int ora_linear_q4_exact(const float* x, const void* w, float* y, int M, int K, int N, int kind) {
    if (M <= 0 || N <= 0) return 0;
    const int be = kind_block_elems(kind);
    if (K % be != 0) return -1;
    const u8* p = (const u8*)w;
    const i64 row_bytes = (i64)(K / be) * kind_block_bytes(kind);
#pragma omp parallel for schedule(static) if ((i64)N * K > 65536)
    for (int n = 0; n < N; ++n) {
        std::vector<double> row((size_t)K);
        const u8* wr = p + (i64)n * row_bytes;
        for (int k = 0; k < K; ++k) row[k] = (double)dequant_one(wr, kind, k);
        for (int m = 0; m < M; ++m) {
            const float* xa = x + (size_t)m * K;
            double acc = 0.0;
            for (int k = 0; k < K; ++k) acc += (double)xa[k] * row[k];
            y[(size_t)m * N + n] = (float)acc;
        }
    }
    return 0;
}

// fp16 weights (lm_head / embeddings in quantised models): core/math_cpu.cpp:121-134.
ORA_API void ora_linear_f16(const float* x, const u16* w, float* y, int M, int K, int N) {
#pragma omp parallel for schedule(static) if ((i64)N * K > 65536)
    for (int n = 0; n < N; ++n) {
        const u16* row = w + (size_t)n * K;
        for (int m = 0; m < M; ++m) {
            const float* xa = x + (size_t)m * K;
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += xa[k] * f16_bits_to_f32(row[k]);
            y[(size_t)m * N + n] = acc;
        }
    }
}

// fp32 weights: core/math_cpu.cpp:117-119 (cpu::gemm with B transposed).  The
// reference sums with a 4x8-lane AVX2 tree or a scalar chain depending on the
// host; this oracle uses the plain scalar chain, the checks are by tolerance.
ORA_API void ora_linear_f32(const float* x, const float* w, float* y, int M, int K, int N) {
#pragma omp parallel for schedule(static) if ((i64)N * K > 65536)
    for (int n = 0; n < N; ++n) {
        const float* row = w + (size_t)n * K;
        for (int m = 0; m < M; ++m) {
            const float* xa = x + (size_t)m * K;
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += xa[k] * row[k];
            y[(size_t)m * N + n] = acc;
        }
    }
}

// A weight handle the layer oracles use: fp32, fp16 or packed.
// wkind: -2 = fp32, -1 = fp16, 0..3 = packed.
static void weight_rows_to_f32(const void* w, int wkind, i64 row0, int rows, int K, float* dst) {
    if (wkind == -2) {
        std::memcpy(dst, (const float*)w + row0 * K, sizeof(float) * (size_t)rows * K);
    } else if (wkind == -1) {
        const u16* p = (const u16*)w + row0 * K;
        for (i64 i = 0; i < (i64)rows * K; ++i) dst[i] = f16_bits_to_f32(p[i]);
    } else {
        const u8* p = (const u8*)w;
        const int be = kind_block_elems(wkind);
        const i64 row_bytes = (i64)(K / be) * kind_block_bytes(wkind);
        for (int r = 0; r < rows; ++r) {
            const u8* wr = p + (row0 + r) * row_bytes;
            for (int k = 0; k < K; ++k)
                dst[(size_t)r * K + k] = weight_value(wr, wkind, k);
        }
    }
}

static void matvec_rows(const float* x, const float* wf, float* y, int K, int N) {
    for (int n = 0; n < N; ++n) {
        const float* row = wf + (size_t)n * K;
        float acc = 0.0f;
        for (int k = 0; k < K; ++k) acc += x[k] * row[k];
        y[n] = acc;
    }
}

// Generic linear over a weight handle.
ORA_API int ora_linear_any(const float* x, const void* w, int wkind, float* y, int M, int K, int N) {
    if (wkind == -2) { ora_linear_f32(x, (const float*)w, y, M, K, N); return 0; }
    if (wkind == -1) { ora_linear_f16(x, (const u16*)w, y, M, K, N); return 0; }
    return ora_linear_q4(x, w, y, M, K, N, wkind);
}

// ----------------------------------------------------------------------------
// Small ops.
// ----------------------------------------------------------------------------

// core/math_cpu.cpp:213-241.  Out-of-range ids give a zero row.
ORA_API void ora_embedding(const i32* ids, const void* table, int half, float* out,
                           i64 ntok, int dim, int vocab) {
    for (i64 t = 0; t < ntok; ++t) {
        float* o = out + t * dim;
        const i32 id = ids[t];
        if (id < 0 || id >= vocab) { std::fill(o, o + dim, 0.0f); continue; }
        if (half) {
            const u16* row = (const u16*)table + (size_t)id * dim;
            for (int i = 0; i < dim; ++i) o[i] = f16_bits_to_f32(row[i]);
        } else {
            std::memcpy(o, (const float*)table + (size_t)id * dim, sizeof(float) * (size_t)dim);
        }
    }
}

// core/math_cpu.cpp:299-316: sum of squares in double, inv = 1/sqrt(mean+eps) in
// double then rounded to float; a non-finite inv becomes 0.
ORA_API void ora_rmsnorm(const float* x, const float* weight, float* out, float* rrms,
                         i64 rows, int dim, float eps) {
    for (i64 r = 0; r < rows; ++r) {
        const float* xr = x + r * dim;
        double ss = 0.0;
        for (int i = 0; i < dim; ++i) ss += (double)xr[i] * xr[i];
        const double inv_d = 1.0 / std::sqrt(ss / (double)dim + (double)eps);
        const float inv = std::isfinite(inv_d) ? (float)inv_d : 0.0f;
        if (rrms) rrms[r] = inv;
        float* o = out + r * dim;
        for (int i = 0; i < dim; ++i) o[i] = xr[i] * inv * weight[i];
    }
}

// core/math_cpu.cpp:464-496: angle = float(double(pos) * double(inv_freq[i])),
// rope_type 1 pairs (i, i+hd/2), otherwise (2i, 2i+1).
static inline void rotate_pair(float& a, float& b, float c, float s) {
    const float a0 = a, b0 = b;
    a = a0 * c - b0 * s;
    b = a0 * s + b0 * c;
}
ORA_API void ora_rope_cached(float* q, float* k, const i32* pos, const float* inv_freq,
                             i64 ntok, int n_heads, int n_kv, int head_dim, int rope_type) {
    const int half = head_dim / 2;
    for (i64 t = 0; t < ntok; ++t) {
        const double p = (double)pos[t];
        for (int i = 0; i < half; ++i) {
            const float ang = (float)(p * (double)inv_freq[i]);
            const float c = std::cos(ang), s = std::sin(ang);
            for (int pass = 0; pass < 2; ++pass) {
                float* base = pass == 0 ? q : k;
                const int nh = pass == 0 ? n_heads : n_kv;
                if (!base) continue;
                for (int h = 0; h < nh; ++h) {
                    float* row = base + (t * nh + h) * head_dim;
                    if (rope_type == 1) rotate_pair(row[i], row[i + half], c, s);
                    else rotate_pair(row[2 * i], row[2 * i + 1], c, s);
                }
            }
        }
    }
}

static inline float silu_f(float v) { return v / (1.0f + std::exp(-v)); }

// core/math_cpu.cpp:537-544.
ORA_API void ora_swiglu(const float* g, const float* u, float* out, i64 n) {
    for (i64 i = 0; i < n; ++i) out[i] = silu_f(g[i]) * u[i];
}

// core/math_cpu.cpp:546-558.
static void softmax_inplace(float* v, int n) {
    if (n <= 0) return;
    float mx = v[0];
    for (int i = 1; i < n; ++i) mx = std::max(mx, v[i]);
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) { v[i] = std::exp(v[i] - mx); sum += v[i]; }
    const float inv = sum > 1e-12f ? 1.0f / sum : 0.0f;
    for (int i = 0; i < n; ++i) v[i] *= inv;
}

// core/math_cpu.cpp:709-722: greedy pick, ties to the lowest id, non-finite
// logits skipped unless every logit is non-finite.
ORA_API i32 ora_argmax(const float* logits, int V) {
    int best = -1;
    float bv = -std::numeric_limits<float>::infinity();
    for (int i = 0; i < V; ++i) {
        const float v = logits[i];
        if (std::isfinite(v) && (best < 0 || v > bv)) { bv = v; best = i; }
    }
    if (best < 0) {
        best = 0;
        for (int i = 1; i < V; ++i) if (logits[i] > logits[best]) best = i;
    }
    return best;
}

// core/math_cpu.cpp:695-707: K largest, ties to the lower id.
ORA_API void ora_topk(const float* logits, int V, int K, float* out_vals, i32* out_ids) {
    std::vector<int> order((size_t)V);
    for (int i = 0; i < V; ++i) order[i] = i;
    std::partial_sort(order.begin(), order.begin() + K, order.end(), [&](int a, int b) {
        if (logits[a] != logits[b]) return logits[a] > logits[b];
        return a < b;
    });
    for (int k = 0; k < K; ++k) { out_vals[k] = logits[order[k]]; out_ids[k] = order[k]; }
}

// core/math_cpu.cpp:724-753: repetition / frequency / presence penalties applied
// once per distinct history token.
ORA_API void ora_rep_penalties(float* logits, int V, const i32* hist, int hist_n,
                               float rep, float freq, float pres) {
    if (hist_n <= 0 || V <= 0) return;
    const bool use_rep = rep > 0.0f && rep != 1.0f;
    if (!use_rep && freq == 0.0f && pres == 0.0f) return;
    std::vector<int> count((size_t)V, 0);
    for (int i = 0; i < hist_n; ++i) if (hist[i] >= 0 && hist[i] < V) ++count[hist[i]];
    for (int t = 0; t < V; ++t) {
        if (!count[t]) continue;
        float& l = logits[t];
        if (use_rep) l = (l > 0.0f) ? l / rep : l * rep;
        if (freq != 0.0f) l -= freq * (float)count[t];
        if (pres != 0.0f) l -= pres;
    }
}

// ----------------------------------------------------------------------------
// Sampling tail: the generator (core/rng.h:8-45), the sampler (inference/sampler.cpp)
// and the cross-entropy used for perplexity (core/math_cpu.cpp:560-612, forward part).
// ----------------------------------------------------------------------------

// core/rng.h:12-22: four splitmix64 outputs of the running seed fill the state.
ORA_API void ora_rng_seed(u64 seed, u64* s) {
    for (int i = 0; i < 4; ++i) {
        seed += 0x9E3779B97F4A7C15ULL;
        u64 z = seed;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
        s[i] = z ^ (z >> 31);
    }
}
static inline u64 rotl64(u64 x, int k) { return (x << k) | (x >> (64 - k)); }
// core/rng.h:24-35 (xoshiro256**).
ORA_API u64 ora_rng_next(u64* s) {
    const u64 r = rotl64(s[1] * 5, 7) * 9;
    const u64 t = s[1] << 17;
    s[2] ^= s[0];
    s[3] ^= s[1];
    s[1] ^= s[2];
    s[0] ^= s[3];
    s[2] ^= t;
    s[3] = rotl64(s[3], 45);
    return r;
}
// core/rng.h:39-41: the top 24 bits as a float in [0, 1).
ORA_API float ora_rng_uniform(u64* s) { return (float)((ora_rng_next(s) >> 40) * (1.0 / 16777216.0)); }

// SamplingConfig::validate, inference/sampler.cpp:36-73.  cfg = {temperature, top_p, min_p,
// repetition_penalty, frequency_penalty, presence_penalty}, icfg = {top_k, repetition_window,
// no_repeat_ngram, greedy}.
ORA_API void ora_sampling_validate(float* f, int* ic) {
    if (!std::isfinite(f[0]) || f[0] < 0.0f) f[0] = 0.0f;
    if (f[0] > 5.0f) f[0] = 5.0f;
    if (!std::isfinite(f[1]) || f[1] < 0.0f) f[1] = 1.0f;
    if (f[1] > 1.0f) f[1] = 1.0f;
    if (!std::isfinite(f[2]) || f[2] < 0.0f) f[2] = 0.0f;
    if (f[2] >= 1.0f) f[2] = 0.0f;
    if (ic[0] < 0) ic[0] = 0;
    if (ic[0] > 2048) ic[0] = 2048;
    if (!std::isfinite(f[3]) || f[3] <= 0.0f) f[3] = 1.0f;
    if (f[3] > 5.0f) f[3] = 5.0f;
    if (!std::isfinite(f[4])) f[4] = 0.0f;
    if (!std::isfinite(f[5])) f[5] = 0.0f;
    f[4] = std::min(5.0f, std::max(-5.0f, f[4]));
    f[5] = std::min(5.0f, std::max(-5.0f, f[5]));
    ic[1] = std::min(8192, std::max(0, ic[1]));
    if (ic[2] < 0) ic[2] = 0;
    if (ic[2] == 1) ic[2] = 2;
    if (ic[2] > 8) ic[2] = 8;
}

namespace {
struct Cand { float v; i32 id; };
// Candidates in descending value; equal values by ascending id (the reference's std::sort
// leaves the order of equal values unspecified; this is the order the device uses).
void sort_candidates(std::vector<Cand>& c) {
    std::sort(c.begin(), c.end(), [](const Cand& a, const Cand& b) { return a.v != b.v ? a.v > b.v : a.id < b.id; });
}
// Sampler::draw_from_scratch, inference/sampler.cpp:206-266.
i32 draw_sorted(const std::vector<Cand>& c, float temperature, float top_p, float min_p, u64* rng) {
    if (!(temperature > 0.0f)) return c[0].id;
    const float inv_t = 1.0f / temperature;
    const float mx = c[0].v;
    std::vector<double> probs(c.size());
    double sum = 0.0;
    for (size_t i = 0; i < c.size(); ++i) {
        probs[i] = std::exp((double)((c[i].v - mx) * inv_t));
        sum += probs[i];
    }
    if (!std::isfinite(sum) || sum <= 0.0) return c[0].id;
    for (size_t i = 0; i < c.size(); ++i) probs[i] /= sum;
    size_t limit = c.size();
    if (min_p > 0.0f) {
        const double thresh = min_p * probs[0];
        size_t n = 0;
        while (n < c.size() && probs[n] >= thresh) ++n;
        limit = std::max<size_t>(1, n);
    }
    if (top_p > 0.0f && top_p < 1.0f) {
        double cum = 0.0;
        size_t n = 0;
        while (n < limit) {
            cum += probs[n];
            ++n;
            if (cum >= (double)top_p) break;
        }
        limit = std::max<size_t>(1, n);
    }
    double renorm = 0.0;
    for (size_t i = 0; i < limit; ++i) renorm += probs[i];
    const double r = (double)ora_rng_uniform(rng) * renorm;
    double acc = 0.0;
    for (size_t i = 0; i < limit; ++i) {
        acc += probs[i];
        if (r <= acc) return c[i].id;
    }
    return c[limit - 1].id;
}
}  // namespace

// Sampler::sample_candidates, inference/sampler.cpp:194-204: the device top-K, sorted, drawn.
ORA_API i32 ora_sample_candidates(const float* vals, const i32* ids, int K, float temperature, float top_p,
                                  float min_p, u64* rng) {
    std::vector<Cand> c((size_t)K);
    for (int i = 0; i < K; ++i) c[i] = Cand{vals[i], ids[i]};
    sort_candidates(c);
    return draw_sorted(c, temperature, top_p, min_p, rng);
}

// Sampler::sample, inference/sampler.cpp:126-192 (with apply_penalties :75-107 and
// ban_no_repeat_ngram :109-124).  The logits are modified in place like the reference's.
// f / ic as in ora_sampling_validate (already validated).
ORA_API i32 ora_sample(float* logits, int vocab, const i32* hist, int nh, const float* f, const int* ic, u64* rng) {
    const float temperature = f[0], top_p = f[1], min_p = f[2], rep_pen = f[3], freq_pen = f[4], pres_pen = f[5];
    const int top_k = ic[0], window_cfg = ic[1], ngram = ic[2], greedy = ic[3];
    const bool rep = rep_pen != 1.0f, freq = freq_pen != 0.0f, pres = pres_pen != 0.0f;
    if (nh > 0 && (rep || freq || pres)) {
        const int window = window_cfg > 0 ? std::min(nh, window_cfg) : nh;
        std::vector<i32> win;
        for (int i = nh - window; i < nh; ++i)
            if (hist[i] >= 0 && hist[i] < vocab) win.push_back(hist[i]);
        std::sort(win.begin(), win.end());
        for (size_t i = 0; i < win.size();) {
            size_t j = i + 1;
            while (j < win.size() && win[j] == win[i]) ++j;
            float& l = logits[win[i]];
            if (rep) l = (l > 0.0f) ? l / rep_pen : l * rep_pen;
            if (freq) l -= freq_pen * (float)(j - i);
            if (pres) l -= pres_pen;
            i = j;
        }
    }
    if (ngram > 0 && nh >= ngram - 1) {
        const int pre = ngram - 1;
        for (int i = 0; i + ngram <= nh; ++i) {
            bool match = true;
            for (int k = 0; k < pre; ++k)
                if (hist[i + k] != hist[nh - pre + k]) { match = false; break; }
            if (!match) continue;
            const i32 nxt = hist[i + pre];
            if (nxt >= 0 && nxt < vocab) logits[nxt] = -1e30f;
        }
    }
    if (greedy || temperature <= 0.0f || top_k == 1) return ora_argmax(logits, vocab);
    const bool no_filter = (top_k <= 0 || top_k >= vocab) && (top_p <= 0.0f || top_p >= 1.0f) && min_p <= 0.0f;
    if (no_filter) {
        // the largest logit (first of equals) changes places with element 0, then one pass
        std::vector<Cand> c((size_t)vocab);
        for (int i = 0; i < vocab; ++i) c[i] = Cand{logits[i], i};
        size_t bi = 0;
        for (size_t i = 1; i < c.size(); ++i)
            if (c[i].v > c[bi].v) bi = i;
        if (bi != 0) std::swap(c[0], c[bi]);
        const float inv_t = 1.0f / temperature;
        const float mx = c[0].v;
        std::vector<double> probs(c.size());
        double sum = 0.0;
        for (size_t i = 0; i < c.size(); ++i) {
            probs[i] = std::exp((double)((c[i].v - mx) * inv_t));
            sum += probs[i];
        }
        if (!std::isfinite(sum) || sum <= 0.0) return c[0].id;
        const double r = (double)ora_rng_uniform(rng) * sum;
        double acc = 0.0;
        for (size_t i = 0; i < c.size(); ++i) {
            acc += probs[i];
            if (r <= acc) return c[i].id;
        }
        return c.back().id;
    }
    const int k = (top_k > 0 && top_k < vocab) ? top_k : vocab;
    std::vector<Cand> c((size_t)vocab);
    for (int i = 0; i < vocab; ++i) c[i] = Cand{logits[i], i};
    sort_candidates(c);
    c.resize((size_t)k);
    return draw_sorted(c, temperature, top_p, min_p, rng);
}

// core/math_cpu.cpp:560-612, forward part: rows with a target in [0, V) contribute
// logZ - logit[target] (+ z_scale * logZ^2), everything accumulated in double.
ORA_API void ora_softmax_cross_entropy(const float* logits, const i32* targets, i64 n, int V, float z_scale,
                                       double* loss_sum, i64* count) {
    double total = 0.0;
    i64 cnt = 0;
    for (i64 i = 0; i < n; ++i) {
        const i32 tgt = targets[i];
        if (tgt < 0 || tgt >= V) continue;
        ++cnt;
        const float* row = logits + i * V;
        float mx = row[0];
        for (int j = 1; j < V; ++j) mx = std::max(mx, row[j]);
        double sum = 0.0;
        for (int j = 0; j < V; ++j) sum += std::exp((double)(row[j] - mx));
        const double logZ = std::log(sum) + (double)mx;
        total += logZ - (double)row[tgt];
        if (z_scale != 0.0f) total += (double)z_scale * logZ * logZ;
    }
    *loss_sum = total;
    *count = cnt;
}

// ----------------------------------------------------------------------------
// MoE.  core/moe_cpu.cpp:198-288 (moe_forward_bias) with the per-token arrays
// widened (the reference stops at ne <= 64, K <= 8).
// ----------------------------------------------------------------------------

// core/moe_cpu.cpp:76-83.  The grouping of four products per step is part of the
// result: ((a0b0 + a1b1) + a2b2) + a3b3 is formed first, then added to the sum.
static inline float router_dot(const float* a, const float* b, int n) {
    float s = 0.0f;
    int i = 0;
    for (; i + 4 <= n; i += 4) {
        float g = a[i] * b[i] + a[i + 1] * b[i + 1];
        g = g + a[i + 2] * b[i + 2];
        g = g + a[i + 3] * b[i + 3];
        s += g;
    }
    for (; i < n; ++i) s += a[i] * b[i];
    return s;
}

// Router for one token: probabilities, K selected experts and mixture weights.
// Selection is on probs + bias (bias may be null), strict '>' scanning experts in
// ascending order so ties go to the lowest index (core/moe_cpu.cpp:85-98);
// mixture weights are the unbiased probs renormalised, or uniform when their sum
// is <= 1e-8 (core/moe_cpu.cpp:244-254).
static void route_token(const float* xt, const float* router_w, const float* bias,
                        int d, int ne, int K, float* probs, i32* idx, float* w) {
    for (int e = 0; e < ne; ++e) probs[e] = router_dot(xt, router_w + (size_t)e * d, d);
    softmax_inplace(probs, ne);
    std::vector<float> sel((size_t)ne);
    for (int e = 0; e < ne; ++e) sel[e] = probs[e] + (bias ? bias[e] : 0.0f);
    for (int k = 0; k < K; ++k) {
        int best = -1;
        float bv = -1e30f;
        for (int e = 0; e < ne; ++e) {
            bool taken = false;
            for (int j = 0; j < k; ++j) if (idx[j] == e) { taken = true; break; }
            if (!taken && sel[e] > bv) { bv = sel[e]; best = e; }
        }
        if (best < 0) best = 0;
        idx[k] = best;
    }
    float sum_w = 0.0f;
    for (int k = 0; k < K; ++k) { w[k] = probs[idx[k]]; sum_w += w[k]; }
    if (sum_w > 1e-8f) {
        const float inv = 1.0f / sum_w;
        for (int k = 0; k < K; ++k) w[k] *= inv;
    } else {
        for (int k = 0; k < K; ++k) w[k] = 1.0f / (float)K;
    }
}

ORA_API void ora_moe_route(const float* x, const float* router_w, const float* router_bias,
                           float* probs, i32* idx, float* w, i64 N, int d, int ne, int K) {
#pragma omp parallel for schedule(static) if (N > 4)
    for (i64 t = 0; t < N; ++t) {
        std::vector<float> p((size_t)ne);
        route_token(x + t * d, router_w, router_bias, d, ne, K, p.data(), idx + t * K, w + t * K);
        if (probs) std::memcpy(probs + t * ne, p.data(), sizeof(float) * (size_t)ne);
    }
}

// Canonical expert grouping: stable counting sort of slot ids s = t*K + k by
// expert (ascending s inside an expert); offsets = exclusive prefix sum of the
// per-expert counts.  The reference CPU path has no permutation and its CUDA path
// (cuda/moe.cu:623-651) orders slots by atomics, so this is the definition the
// CUDA library is held to.
ORA_API void ora_moe_permutation(const i32* idx, i64 NK, int ne, i32* grouped, i32* offsets) {
    std::vector<i64> count((size_t)ne + 1, 0);
    for (i64 s = 0; s < NK; ++s) ++count[(size_t)idx[s] + 1];
    for (int e = 0; e < ne; ++e) count[e + 1] += count[e];
    for (int e = 0; e <= ne; ++e) offsets[e] = (i32)count[e];
    std::vector<i64> cursor(count.begin(), count.end() - 1);
    for (i64 s = 0; s < NK; ++s) grouped[cursor[idx[s]]++] = (i32)s;
}

// Whole MoE layer.  wkind selects the storage of the six expert matrices
// (-2 fp32, -1 fp16, 0..3 packed).  Packed / fp16 experts go through the fp16
// value exactly as the reference does (core/moe_cpu.cpp:290-313 after
// ops::quant_materialize).  gates/ups: [ne*E, d]; downs: [ne*d, E]; shared:
// [SH,d],[SH,d],[d,SH] (may be null).  Optional outputs may be null.
ORA_API int ora_moe_forward(const float* x, const float* router_w, const float* router_bias,
                            const void* gates, const void* ups, const void* downs,
                            const void* sh_g, const void* sh_u, const void* sh_d,
                            float* out, float* probs_cache, i32* idx_cache, float* w_cache,
                            i64 N, int d, int E, int ne, int K, int SH, int wkind) {
    if (N <= 0) return 0;
    if (K < 1 || ne < 1 || K > ne || d < 1 || E < 1) return -1;
    std::vector<i32> idx((size_t)N * K);
    std::vector<float> w((size_t)N * K);
    ora_moe_route(x, router_w, router_bias, probs_cache, idx.data(), w.data(), N, d, ne, K);
    if (idx_cache) std::memcpy(idx_cache, idx.data(), sizeof(i32) * idx.size());
    if (w_cache) std::memcpy(w_cache, w.data(), sizeof(float) * w.size());

    // shared expert first: it initialises out (core/moe_cpu.cpp:260-267)
    const bool has_shared = sh_g && sh_u && sh_d && SH > 0;
    if (has_shared) {
        std::vector<float> g((size_t)SH * d), u((size_t)SH * d), dn((size_t)d * SH);
        weight_rows_to_f32(sh_g, wkind, 0, SH, d, g.data());
        weight_rows_to_f32(sh_u, wkind, 0, SH, d, u.data());
        weight_rows_to_f32(sh_d, wkind, 0, d, SH, dn.data());
#pragma omp parallel for schedule(static) if (N > 4)
        for (i64 t = 0; t < N; ++t) {
            std::vector<float> a((size_t)SH), b((size_t)SH);
            matvec_rows(x + t * d, g.data(), a.data(), d, SH);
            matvec_rows(x + t * d, u.data(), b.data(), d, SH);
            for (int i = 0; i < SH; ++i) a[i] = silu_f(a[i]) * b[i];
            matvec_rows(a.data(), dn.data(), out + t * d, SH, d);
        }
    } else {
        std::fill(out, out + N * d, 0.0f);
    }

    // routed experts, expert-major so each expert is widened once; a token's K
    // contributions are still added in k order (core/moe_cpu.cpp:269-286).
    std::vector<float> contrib((size_t)N * K * d);
    std::vector<i32> grouped((size_t)N * K), offsets((size_t)ne + 1);
    ora_moe_permutation(idx.data(), N * K, ne, grouped.data(), offsets.data());
#pragma omp parallel for schedule(dynamic)
    for (int e = 0; e < ne; ++e) {
        if (offsets[e + 1] == offsets[e]) continue;
        std::vector<float> g((size_t)E * d), u((size_t)E * d), dn((size_t)d * E);
        weight_rows_to_f32(gates, wkind, (i64)e * E, E, d, g.data());
        weight_rows_to_f32(ups, wkind, (i64)e * E, E, d, u.data());
        weight_rows_to_f32(downs, wkind, (i64)e * d, d, E, dn.data());
        std::vector<float> a((size_t)E), b((size_t)E);
        for (i32 p = offsets[e]; p < offsets[e + 1]; ++p) {
            const i32 s = grouped[p];
            const float* xt = x + (i64)(s / K) * d;
            matvec_rows(xt, g.data(), a.data(), d, E);
            matvec_rows(xt, u.data(), b.data(), d, E);
            for (int i = 0; i < E; ++i) a[i] = silu_f(a[i]) * b[i];
            matvec_rows(a.data(), dn.data(), contrib.data() + (size_t)s * d, E, d);
        }
    }
    for (i64 t = 0; t < N; ++t)
        for (int k = 0; k < K; ++k) {
            const float wk = w[t * K + k];
            const float* c = contrib.data() + (size_t)(t * K + k) * d;
            float* o = out + t * d;
            for (int j = 0; j < d; ++j) o[j] += wk * c[j];
        }
    return 0;
}

// ----------------------------------------------------------------------------
// Mamba-2.
// ----------------------------------------------------------------------------
static inline float softplus20(float u) { return u > 20.0f ? u : std::log1p(std::exp(u)); }

// Conv + scan + gated norm over already projected rows (no in/out projection):
// the middle of core/mamba_cpu.cpp:81-194.  proj: [B*T, proj_size] rows laid out
// gate(d_inner) | bc(conv_dim) | dt(n_heads); conv_state (optional, [B, conv_dim,
// k-1], oldest first) seeds the window and receives the last k-1 raw inputs -
// null reproduces the reference's zero-initialised window; state [B, n_heads,
// d_head, d_state] is carried; normed: [B*T, d_inner].
ORA_API int ora_mamba2_core(const float* proj, const float* conv_w, const float* conv_b,
                            const float* dt_bias, const float* a_log, const float* Dv,
                            const float* norm_w, float* conv_state, float* state, float* normed,
                            int B, int T, int d_inner, int conv_dim, int n_heads, int d_head,
                            int d_state, int k, float eps) {
    const int proj_size = d_inner + conv_dim + n_heads;
    const int tot = (conv_dim - d_inner) / 2;
    if (tot < d_state || tot % d_state != 0) return -1;
    const int groups = tot / d_state;
    if (n_heads % groups != 0) return -1;
    const int hpg = n_heads / groups;
    const int win = k > 1 ? k - 1 : 1;
    const i64 NT = (i64)B * T;
    std::vector<float> bc((size_t)NT * conv_dim);
#pragma omp parallel for schedule(static)
    for (int c = 0; c < conv_dim; ++c) {
        std::vector<float> wv((size_t)win);
        const float* wc = conv_w + (size_t)c * k;
        const float bias = conv_b ? conv_b[c] : 0.0f;
        for (int b = 0; b < B; ++b) {
            for (int j = 0; j < win; ++j)
                wv[j] = conv_state ? conv_state[((size_t)b * conv_dim + c) * win + j] : 0.0f;
            for (int t = 0; t < T; ++t) {
                const float raw = proj[((size_t)b * T + t) * proj_size + d_inner + c];
                float acc = bias;
                for (int j = 0; j < k; ++j) acc += wc[j] * (j == k - 1 ? raw : wv[j]);
                bc[((size_t)b * T + t) * conv_dim + c] = silu_f(acc);
                for (int j = 0; j + 1 < win; ++j) wv[j] = wv[j + 1];
                wv[win - 1] = raw;
            }
            if (conv_state)
                for (int j = 0; j < win; ++j) conv_state[((size_t)b * conv_dim + c) * win + j] = wv[j];
        }
    }
    const int inner = n_heads * d_head;
    std::vector<float> y((size_t)NT * d_inner);
#pragma omp parallel for schedule(static)
    for (int row = 0; row < B * inner; ++row) {
        const int b = row / inner, rem = row % inner, h = rem / d_head;
        const float a = -std::exp(a_log[h]);
        float* srow = state + (size_t)row * d_state;
        const int goff = (h / hpg) * d_state;
        for (int t = 0; t < T; ++t) {
            const float* prow = proj + ((size_t)b * T + t) * proj_size;
            const float* brow = bc.data() + ((size_t)b * T + t) * conv_dim;
            const float dt = softplus20(prow[proj_size - n_heads + h] + dt_bias[h]);
            const float dA = std::exp(a * dt);
            const float xv = brow[rem];
            float acc = 0.0f;
            for (int j = 0; j < d_state; ++j) {
                srow[j] = dA * srow[j] + (dt * brow[d_inner + goff + j]) * xv;
                acc += brow[d_inner + tot + goff + j] * srow[j];
            }
            y[((size_t)b * T + t) * d_inner + rem] = acc + Dv[h] * xv;
        }
    }
#pragma omp parallel for schedule(static)
    for (i64 n = 0; n < NT; ++n) {
        const float* yr = y.data() + (size_t)n * d_inner;
        const float* gr = proj + (size_t)n * proj_size;
        float* o = normed + (size_t)n * d_inner;
        double var = 0.0;
        for (int c = 0; c < d_inner; ++c) {
            const float v = yr[c] * silu_f(gr[c]);
            o[c] = v;
            var += (double)v * v;
        }
        var /= (double)d_inner;
        const float inv = 1.0f / std::sqrt((float)var + eps);
        for (int c = 0; c < d_inner; ++c) o[c] = o[c] * inv * norm_w[c];
    }
    return 0;
}

// Whole layer over [B,T] (core/mamba_cpu.cpp:48-198): in_proj, conv (window
// zero-initialised on every call), scan with carried state, gated norm, out_proj.
ORA_API int ora_mamba2_forward(const float* x, const void* w_in, const float* conv_w,
                               const float* conv_b, const float* dt_bias, const float* a_log,
                               const float* Dv, const float* norm_w, const void* w_out,
                               float* state, float* out, int B, int T, int d, int d_inner,
                               int conv_dim, int n_heads, int d_head, int d_state, int k,
                               float eps, int wkind) {
    if (B <= 0 || T <= 0) return 0;
    const int proj_size = d_inner + conv_dim + n_heads;
    const i64 NT = (i64)B * T;
    std::vector<float> proj((size_t)NT * proj_size), normed((size_t)NT * d_inner);
    if (ora_linear_any(x, w_in, wkind, proj.data(), (int)NT, d, proj_size)) return -1;
    if (ora_mamba2_core(proj.data(), conv_w, conv_b, dt_bias, a_log, Dv, norm_w, nullptr, state,
                        normed.data(), B, T, d_inner, conv_dim, n_heads, d_head, d_state, k, eps))
        return -1;
    return ora_linear_any(normed.data(), w_out, wkind, out, (int)NT, d_inner, d);
}

// One decode token with the carried conv window [conv_dim, k-1] (oldest first)
// and ssm state [n_heads*d_head, d_state]: the host path of
// Generator::decode_mamba_layer, inference/generator.cpp:510-616.
ORA_API int ora_mamba2_step(const float* x, const void* w_in, const float* conv_w,
                            const float* conv_b, const float* dt_bias, const float* a_log,
                            const float* Dv, const float* norm_w, const void* w_out,
                            float* conv_state, float* ssm_state, float* out, int d, int d_inner,
                            int conv_dim, int n_heads, int d_head, int d_state, int k, float eps,
                            int wkind) {
    const int proj_size = d_inner + conv_dim + n_heads;
    std::vector<float> proj((size_t)proj_size), normed((size_t)d_inner);
    if (ora_linear_any(x, w_in, wkind, proj.data(), 1, d, proj_size)) return -1;
    if (ora_mamba2_core(proj.data(), conv_w, conv_b, dt_bias, a_log, Dv, norm_w, conv_state,
                        ssm_state, normed.data(), 1, 1, d_inner, conv_dim, n_heads, d_head,
                        d_state, k, eps))
        return -1;
    return ora_linear_any(normed.data(), w_out, wkind, out, 1, d_inner, d);
}

// ----------------------------------------------------------------------------
// Attention.
// ----------------------------------------------------------------------------

// Prefill: causal, optional sliding window and segment mask
// (core/attn_cpu.cpp:29-94).  q [B,T,H,hd], k/v [B,T,KV,hd], out [B,T,H,hd];
// probs ([B,H,T,T]) optional.
ORA_API void ora_attention_forward(const float* q, const float* k, const float* v, float* out,
                                   float* probs, int B, int T, int H, int KV, int hd,
                                   float scale, int window, const i32* segment_ids) {
    const int group = H / KV;
    const size_t qs = (size_t)T * H * hd, kvs = (size_t)T * KV * hd;
#pragma omp parallel for schedule(static)
    for (int bh = 0; bh < B * H; ++bh) {
        const int b = bh / H, h = bh % H, kvh = h / group;
        std::vector<float> s((size_t)T);
        for (int t = 0; t < T; ++t) {
            const float* qh = q + b * qs + ((size_t)t * H + h) * hd;
            const int j0 = window > 0 ? std::max(0, t - window + 1) : 0;
            const int len = t + 1 - j0;
            const i32 seg_t = segment_ids ? segment_ids[(size_t)b * T + t] : 0;
            float mx = -3.4e38f;
            for (int j = j0; j <= t; ++j) {
                if (segment_ids && seg_t >= 0 && segment_ids[(size_t)b * T + j] != seg_t) {
                    s[j - j0] = -3.4e38f;
                    continue;
                }
                const float* kh = k + b * kvs + ((size_t)j * KV + kvh) * hd;
                float dot = 0.0f;
                for (int c = 0; c < hd; ++c) dot += qh[c] * kh[c];
                dot *= scale;
                s[j - j0] = dot;
                mx = std::max(mx, dot);
            }
            float sum = 0.0f;
            for (int j = 0; j < len; ++j) {
                s[j] = s[j] < -3.0e38f ? 0.0f : std::exp(s[j] - mx);
                sum += s[j];
            }
            const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
            float* o = out + b * qs + ((size_t)t * H + h) * hd;
            std::fill(o, o + hd, 0.0f);
            for (int j = 0; j < len; ++j) {
                const float p = s[j] * inv;
                s[j] = p;
                const float* vh = v + b * kvs + ((size_t)(j + j0) * KV + kvh) * hd;
                for (int c = 0; c < hd; ++c) o[c] += p * vh[c];
            }
            if (probs) {
                float* pr = probs + (((size_t)b * H + h) * T + t) * T;
                std::fill(pr, pr + T, 0.0f);
                std::memcpy(pr + j0, s.data(), sizeof(float) * (size_t)len);
            }
        }
    }
}

// Logical position -> physical cache row of the ring cache with a pinned prefix
// (core/attn_cpu.cpp:151-156).
static inline size_t ring_row(int j, int pinned, int ring_start, int ring_cap) {
    if (j < pinned) return (size_t)j;
    const int cap = ring_cap > 0 ? ring_cap : 1;
    return (size_t)pinned + (size_t)((ring_start + (j - pinned)) % cap);
}

// One query token against the ring cache (core/attn_cpu.cpp:158-254).  half != 0:
// the cache holds fp16.  Returns -1 on the argument errors the reference rejects.
ORA_API int ora_attention_decode_ring(const float* q, const void* kcache, const void* vcache,
                                      int half, float* out, int H, int KV, int hd,
                                      int ring_start, int pinned, int cur_len, int cache_max,
                                      float scale, int window) {
    if (H <= 0 || KV <= 0 || hd <= 0 || H % KV != 0) return -1;
    if (cur_len < 0 || cache_max < 0 || cur_len > cache_max) return -1;
    if (pinned < 0 || pinned > cur_len) return -1;
    const int ring_cap = cache_max - pinned;
    if (cur_len > pinned && (ring_cap <= 0 || ring_start < 0 || ring_start >= ring_cap)) return -1;
    const int group = H / KV;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < H; ++h) {
        const int kvh = h / group;
        const float* qh = q + (size_t)h * hd;
        const int j0 = (window > 0 && cur_len > window) ? cur_len - window : 0;
        std::vector<float> s((size_t)std::max(cur_len, 1));
        float mx = -3.4e38f;
        for (int j = j0; j < cur_len; ++j) {
            const size_t row = ring_row(j, pinned, ring_start, ring_cap);
            float dot = 0.0f;
            if (half) {
                const u16* kh = (const u16*)kcache + (row * KV + kvh) * hd;
                for (int c = 0; c < hd; ++c) dot += qh[c] * f16_bits_to_f32(kh[c]);
            } else {
                const float* kh = (const float*)kcache + (row * KV + kvh) * hd;
                for (int c = 0; c < hd; ++c) dot += qh[c] * kh[c];
            }
            dot *= scale;
            s[j] = dot;
            mx = std::max(mx, dot);
        }
        float sum = 0.0f;
        for (int j = j0; j < cur_len; ++j) { s[j] = std::exp(s[j] - mx); sum += s[j]; }
        const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        float* o = out + (size_t)h * hd;
        std::fill(o, o + hd, 0.0f);
        for (int j = j0; j < cur_len; ++j) {
            const size_t row = ring_row(j, pinned, ring_start, ring_cap);
            const float p = s[j] * inv;
            if (half) {
                const u16* vh = (const u16*)vcache + (row * KV + kvh) * hd;
                for (int c = 0; c < hd; ++c) o[c] += p * f16_bits_to_f32(vh[c]);
            } else {
                const float* vh = (const float*)vcache + (row * KV + kvh) * hd;
                for (int c = 0; c < hd; ++c) o[c] += p * vh[c];
            }
        }
    }
    return 0;
}

ORA_API int ora_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
