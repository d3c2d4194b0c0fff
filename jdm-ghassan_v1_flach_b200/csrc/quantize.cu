// Device quantisers: fp32 -> packed blocks, bit-identical to the CPU functions.
// Q8_0 / Q4_0 / Q4_1 follow quantization/quantize.cpp:20-246 of the reference
// (amax/127 or amax/8 or (max-min)/15 scale stored as fp16, lround, clamp; a block
// holding a non-finite value becomes the zero block); Q4_K is this library's own
// single-pass quantiser (per 32 weights: lo = min(x, 0), scale = (max-lo)/15;
// super-block scales max/63 as fp16; 6-bit codes and nibbles by round-half-up).
// One thread per block; every arithmetic step is a single correctly rounded fp32
// operation so the bytes equal the host's.
#include "quant.cuh"

namespace b200 {

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
__device__ __forceinline__ int lround_dev(float v) { return (int)roundf(v); }       // half away from zero
__device__ __forceinline__ int round_half_up(float v) { return (int)floorf(__fadd_rn(v, 0.5f)); }
// every block starts on an even address (block sizes 18/20/34/144, even header offsets)
__device__ __forceinline__ void st16(uint8_t* p, uint16_t v) { *reinterpret_cast<uint16_t*>(p) = v; }

template <int KIND>
__global__ void __launch_bounds__(128) quantize_kernel(const float* __restrict__ src, uint8_t* __restrict__ dst,
                                                       int64_t nblocks) {
    constexpr int BE = KIND == 3 ? 256 : 32;
    constexpr int BB = KIND == 0 ? 18 : KIND == 1 ? 20 : KIND == 2 ? 34 : 144;
    const int64_t b = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const float* x = src + b * BE;
    uint8_t* o = dst + b * BB;
    bool bad = false;
    for (int i = 0; i < BE; ++i) bad |= !isfinite(x[i]);
    if (KIND == 2) {
        if (bad) { st16(o, 0); for (int i = 0; i < 32; ++i) o[2 + i] = 0; return; }
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[i]));
        const float scale = __fdiv_rn(amax, 127.0f);
        const float inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
        st16(o, float_to_half_bits(scale));
        for (int i = 0; i < 32; ++i) o[2 + i] = (uint8_t)(int8_t)clampi(lround_dev(__fmul_rn(x[i], inv)), -127, 127);
    } else if (KIND == 0) {
        if (bad) { st16(o, 0); for (int i = 0; i < 16; ++i) o[2 + i] = 0x88; return; }
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[i]));
        const float scale = __fdiv_rn(amax, 8.0f);
        const float inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
        st16(o, float_to_half_bits(scale));
        for (int j = 0; j < 16; ++j) {
            const int lo = clampi(lround_dev(__fmul_rn(x[j], inv)), -8, 7) + 8;
            const int hi = clampi(lround_dev(__fmul_rn(x[j + 16], inv)), -8, 7) + 8;
            o[2 + j] = (uint8_t)((hi << 4) | lo);
        }
    } else if (KIND == 1) {
        if (bad) { for (int i = 0; i < 20; ++i) o[i] = 0; return; }
        float mn = x[0], mx = x[0];
        for (int i = 1; i < 32; ++i) { mn = fminf(mn, x[i]); mx = fmaxf(mx, x[i]); }
        const float scale = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
        const float inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
        st16(o, float_to_half_bits(scale));
        st16(o + 2, float_to_half_bits(mn));
        for (int j = 0; j < 16; ++j) {
            const int lo = clampi(lround_dev(__fmul_rn(__fsub_rn(x[j], mn), inv)), 0, 15);
            const int hi = clampi(lround_dev(__fmul_rn(__fsub_rn(x[j + 16], mn), inv)), 0, 15);
            o[4 + j] = (uint8_t)((hi << 4) | lo);
        }
    } else {
        if (bad) { for (int i = 0; i < 144; ++i) o[i] = 0; return; }
        float sc[8], mnv[8];
        float max_sc = 0.0f, max_mn = 0.0f;
        for (int s = 0; s < 8; ++s) {
            float lo = 0.0f, hi = x[32 * s];
            for (int i = 0; i < 32; ++i) { lo = fminf(lo, x[32 * s + i]); hi = fmaxf(hi, x[32 * s + i]); }
            if (hi < lo) hi = lo;
            sc[s] = __fdiv_rn(__fsub_rn(hi, lo), 15.0f);
            mnv[s] = -lo;
            max_sc = fmaxf(max_sc, sc[s]);
            max_mn = fmaxf(max_mn, mnv[s]);
        }
        const float inv_sc = max_sc > 0.0f ? __fdiv_rn(63.0f, max_sc) : 0.0f;
        const float inv_mn = max_mn > 0.0f ? __fdiv_rn(63.0f, max_mn) : 0.0f;
        int ls[8], lm[8];
        for (int s = 0; s < 8; ++s) {
            ls[s] = clampi(round_half_up(__fmul_rn(inv_sc, sc[s])), 0, 63);
            lm[s] = clampi(round_half_up(__fmul_rn(inv_mn, mnv[s])), 0, 63);
        }
        const uint16_t d16 = float_to_half_bits(__fdiv_rn(max_sc, 63.0f));
        const uint16_t m16 = float_to_half_bits(__fdiv_rn(max_mn, 63.0f));
        st16(o, d16);
        st16(o + 2, m16);
        uint8_t scales[12];
        for (int i = 0; i < 12; ++i) scales[i] = 0;
        for (int j = 0; j < 8; ++j) {
            if (j < 4) {
                scales[j] = (uint8_t)ls[j];
                scales[j + 4] = (uint8_t)lm[j];
            } else {
                scales[j + 4] = (uint8_t)((ls[j] & 0x0F) | ((lm[j] & 0x0F) << 4));
                scales[j - 4] |= (uint8_t)((ls[j] >> 4) << 6);
                scales[j] |= (uint8_t)((lm[j] >> 4) << 6);
            }
        }
        for (int i = 0; i < 12; ++i) o[4 + i] = scales[i];
        const float d = half_bits_to_float(d16), dmin = half_bits_to_float(m16);
        for (int g = 0; g < 4; ++g) {
            const float dd0 = __fmul_rn(d, (float)ls[2 * g]), dm0 = __fmul_rn(dmin, (float)lm[2 * g]);
            const float dd1 = __fmul_rn(d, (float)ls[2 * g + 1]), dm1 = __fmul_rn(dmin, (float)lm[2 * g + 1]);
            for (int l = 0; l < 32; ++l) {
                int q0 = 0, q1 = 0;
                if (dd0 > 0.0f) q0 = clampi(round_half_up(__fdiv_rn(__fadd_rn(x[64 * g + l], dm0), dd0)), 0, 15);
                if (dd1 > 0.0f) q1 = clampi(round_half_up(__fdiv_rn(__fadd_rn(x[64 * g + 32 + l], dm1), dd1)), 0, 15);
                o[16 + 32 * g + l] = (uint8_t)(q0 | (q1 << 4));
            }
        }
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_quantize(const float* src, void* dst, int64_t n, int kind) {
    if (n == 0) return B200_OK;
    B200_REQUIRE(src && dst && n > 0, "quantize: bad arguments");
    B200_REQUIRE(kind >= 0 && kind <= 3, "quantize: unknown kind %d", kind);
    B200_REQUIRE(n % q_block_elems(kind) == 0, "quantize: n must be a multiple of %d", q_block_elems(kind));
    const int64_t nb = n / q_block_elems(kind);
    const unsigned grid = (unsigned)ceil_div64(nb, 128);
    uint8_t* d = static_cast<uint8_t*>(dst);
    switch (kind) {
        case 0: quantize_kernel<0><<<grid, 128, 0, stream()>>>(src, d, nb); break;
        case 1: quantize_kernel<1><<<grid, 128, 0, stream()>>>(src, d, nb); break;
        case 2: quantize_kernel<2><<<grid, 128, 0, stream()>>>(src, d, nb); break;
        default: quantize_kernel<3><<<grid, 128, 0, stream()>>>(src, d, nb); break;
    }
    B200_LAUNCH_CHECK("quantize_kernel");
    return B200_OK;
}
