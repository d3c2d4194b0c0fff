// Device quantisers: fp32 -> packed blocks, bit-identical to the CPU functions.
// Q8_0 / Q4_0 / Q4_1 (kinds 2 / 0 / 1) follow quantization/quantize.cpp:20-246 of the
// reference (amax/127 or amax/8 or (max-min)/15 scale stored as fp16, lround, clamp; a
// block holding a non-finite value becomes the zero block); kind 4 fills the Q4_0 layout
// by the rule of the reference's GGUF writer (format/gguf_codec.cpp:408-460: scale from
// the signed extreme, d = vmax / -8, codes truncated after + 8.5); Q4_K (kind 3) is this
// library's own single-pass quantiser (per 32 weights: lo = min(x, 0), scale =
// (max-lo)/15; super-block scales max/63 as fp16; 6-bit codes and nibbles by
// round-half-up).  Every arithmetic step is a single correctly rounded fp32 operation so
// the bytes equal the host's.
//
// This is the load-time path (an fp32 / fp16 checkpoint quantised on the way in), an HBM
// stream of 4 bytes in per 0.56-1.06 bytes out: eight lanes share a 32-weight block (one
// 128-byte line per block, 16-byte loads), a warp shares a 256-weight Q4_K super-block;
// the few statistics travel by shuffles and the packed bytes leave as whole words.
#include "quant.cuh"

namespace b200 {

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
__device__ __forceinline__ int lround_dev(float v) { return (int)roundf(v); }       // half away from zero
__device__ __forceinline__ int round_half_up(float v) { return (int)floorf(__fadd_rn(v, 0.5f)); }
// every block starts on an even address (block sizes 18/20/34/144, even header offsets)
__device__ __forceinline__ void st16(uint8_t* p, uint16_t v) { *reinterpret_cast<uint16_t*>(p) = v; }
__device__ __forceinline__ void st32_as_16(uint8_t* p, uint32_t v) {       // p even, not always a multiple of 4
    st16(p, (uint16_t)(v & 0xFFFF));
    st16(p + 2, (uint16_t)(v >> 16));
}

// 32-weight blocks: lanes 8g..8g+7 of a warp own block g of the warp's four; lane l of the
// group holds weights 4l..4l+3.
template <int KIND>
__global__ void __launch_bounds__(256) quantize32_kernel(const float* __restrict__ src, uint8_t* __restrict__ dst,
                                                        int64_t nblocks) {
    constexpr int BB = KIND == 1 ? 20 : KIND == 2 ? 34 : 18;
    const int lane = threadIdx.x & 31, l = lane & 7;
    const unsigned gmask = 0xFFu << (lane & 24);
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t b0 = warp * 4; b0 < nblocks; b0 += nwarps * 4) {
        const int64_t b = b0 + (lane >> 3);
        const bool live = b < nblocks;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) v = *reinterpret_cast<const float4*>(src + b * 32 + 4 * l);
        const float x[4] = {v.x, v.y, v.z, v.w};
        uint8_t* o = dst + b * BB;
        bool bad = !(isfinite(x[0]) && isfinite(x[1]) && isfinite(x[2]) && isfinite(x[3]));
        bad = (__ballot_sync(0xffffffffu, bad) & gmask) != 0;
        if (KIND == 2 || KIND == 0) {
            float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
            for (int s = 1; s < 8; s <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
            const float scale = __fdiv_rn(amax, KIND == 2 ? 127.0f : 8.0f);
            const float inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
            int q[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = lround_dev(__fmul_rn(x[i], inv));
                q[i] = KIND == 2 ? clampi(r, -127, 127) : clampi(r, -8, 7) + 8;
            }
            if (KIND == 2) {
                uint32_t w = (uint32_t)(uint8_t)(int8_t)q[0] | ((uint32_t)(uint8_t)(int8_t)q[1] << 8) |
                             ((uint32_t)(uint8_t)(int8_t)q[2] << 16) | ((uint32_t)(uint8_t)(int8_t)q[3] << 24);
                if (bad) w = 0;
                if (live) {
                    if (l == 0) st16(o, bad ? (uint16_t)0 : float_to_half_bits(scale));
                    st32_as_16(o + 2 + 4 * l, w);
                }
            } else {
                // byte j = code(j + 16) << 4 | code(j): lanes 4..7 hand their codes to lanes 0..3
                const uint32_t mine = (uint32_t)q[0] | ((uint32_t)q[1] << 8) | ((uint32_t)q[2] << 16) | ((uint32_t)q[3] << 24);
                const uint32_t hi = __shfl_down_sync(0xffffffffu, mine, 4);
                uint32_t w = mine | (hi << 4);
                if (bad) w = 0x88888888u;
                if (live) {
                    if (l == 0) st16(o, bad ? (uint16_t)0 : float_to_half_bits(scale));
                    if (l < 4) st32_as_16(o + 2 + 4 * l, w);
                }
            }
        } else if (KIND == 4) {
            // the first element of largest magnitude, with its sign
            float amax = 0.0f, vmax = 0.0f;
            int at = 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float a = fabsf(x[i]);
                if (a > amax) { amax = a; vmax = x[i]; at = 4 * l + i; }
            }
#pragma unroll
            for (int s = 1; s < 8; s <<= 1) {
                const float oa = __shfl_xor_sync(0xffffffffu, amax, s), ov = __shfl_xor_sync(0xffffffffu, vmax, s);
                const int oat = __shfl_xor_sync(0xffffffffu, at, s);
                if (oa > amax || (oa == amax && oat < at)) { amax = oa; vmax = ov; at = oat; }
            }
            const bool zero = !isfinite(amax) || amax == 0.0f;
            const float d = __fdiv_rn(vmax, -8.0f);
            const float id = __fdiv_rn(1.0f, d);
            int q[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float f = __fadd_rn(__fmul_rn(x[i], id), 8.5f);
                q[i] = isnan(f) ? 0 : clampi((int)f, 0, 15);
            }
            const uint32_t mine = (uint32_t)q[0] | ((uint32_t)q[1] << 8) | ((uint32_t)q[2] << 16) | ((uint32_t)q[3] << 24);
            const uint32_t hi = __shfl_down_sync(0xffffffffu, mine, 4);
            uint32_t w = mine | (hi << 4);
            if (zero) w = 0x88888888u;
            if (live) {
                if (l == 0) st16(o, zero ? (uint16_t)0 : float_to_half_bits(d));
                if (l < 4) st32_as_16(o + 2 + 4 * l, w);
            }
        } else {   // Q4_1
            float mn = fminf(fminf(x[0], x[1]), fminf(x[2], x[3])), mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
#pragma unroll
            for (int s = 1; s < 8; s <<= 1) {
                mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, s));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
            }
            const float scale = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
            const float inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
            int q[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) q[i] = clampi(lround_dev(__fmul_rn(__fsub_rn(x[i], mn), inv)), 0, 15);
            const uint32_t mine = (uint32_t)q[0] | ((uint32_t)q[1] << 8) | ((uint32_t)q[2] << 16) | ((uint32_t)q[3] << 24);
            const uint32_t hi = __shfl_down_sync(0xffffffffu, mine, 4);
            uint32_t w = mine | (hi << 4);
            if (bad) w = 0;
            if (live) {
                if (l == 0) {
                    st16(o, bad ? (uint16_t)0 : float_to_half_bits(scale));
                    st16(o + 2, bad ? (uint16_t)0 : float_to_half_bits(mn));
                }
                if (l < 4) *reinterpret_cast<uint32_t*>(o + 4 + 4 * l) = w;      // 20 b + 4 + 4 l: a multiple of 4
            }
        }
    }
}

// Q4_K: one warp per 256-weight super-block; lane t holds weights 8t..8t+7 (sub-block t / 4).
__global__ void __launch_bounds__(256) quantize_q4k_kernel(const float* __restrict__ src, uint8_t* __restrict__ dst,
                                                          int64_t nblocks) {
    const int lane = threadIdx.x & 31, sub = lane >> 2;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t b = warp; b < nblocks; b += nwarps) {
        const float4 v0 = *reinterpret_cast<const float4*>(src + b * 256 + 8 * lane);
        const float4 v1 = *reinterpret_cast<const float4*>(src + b * 256 + 8 * lane + 4);
        const float x[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        uint8_t* o = dst + b * 144;
        bool bad = false;
#pragma unroll
        for (int i = 0; i < 8; ++i) bad |= !isfinite(x[i]);
        if (__any_sync(0xffffffffu, bad)) {
            // 144 zero bytes: 36 words
            reinterpret_cast<uint32_t*>(o)[lane] = 0;
            if (lane < 4) reinterpret_cast<uint32_t*>(o)[32 + lane] = 0;
            continue;
        }
        // per sub-block: lo = min(x, 0), hi = max(x) (>= lo)
        float lo = 0.0f, hi = x[0];
#pragma unroll
        for (int i = 0; i < 8; ++i) { lo = fminf(lo, x[i]); hi = fmaxf(hi, x[i]); }
        // the host's loop starts hi at the sub-block's first weight and lo at 0
#pragma unroll
        for (int s = 1; s < 4; s <<= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, s));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, s));
        }
        if (hi < lo) hi = lo;
        const float sc = __fdiv_rn(__fsub_rn(hi, lo), 15.0f), mnv = -lo;
        // the host's running maximum starts at +0: -0 (a sub-block without negatives) must not survive
        float max_sc = sc, max_mn = __fadd_rn(mnv, 0.0f);
#pragma unroll
        for (int s = 4; s < 32; s <<= 1) {
            max_sc = fmaxf(max_sc, __shfl_xor_sync(0xffffffffu, max_sc, s));
            max_mn = fmaxf(max_mn, __shfl_xor_sync(0xffffffffu, max_mn, s));
        }
        const float inv_sc = max_sc > 0.0f ? __fdiv_rn(63.0f, max_sc) : 0.0f;
        const float inv_mn = max_mn > 0.0f ? __fdiv_rn(63.0f, max_mn) : 0.0f;
        const int ls = clampi(round_half_up(__fmul_rn(inv_sc, sc)), 0, 63);
        const int lm = clampi(round_half_up(__fmul_rn(inv_mn, mnv)), 0, 63);
        const uint16_t d16 = float_to_half_bits(__fdiv_rn(max_sc, 63.0f));
        const uint16_t m16 = float_to_half_bits(__fdiv_rn(max_mn, 63.0f));
        // header: d, dmin, then the 12 bytes of 6-bit codes; byte j is built by lane j
        {
            const int j = lane < 12 ? lane : 0;
            const int a = j < 4 ? j : j < 8 ? j - 4 : j - 4;            // sub-block whose code fills the low bits
            const int ls_a = __shfl_sync(0xffffffffu, ls, 4 * a), lm_a = __shfl_sync(0xffffffffu, lm, 4 * a);
            const int hi_sub = j < 4 ? j + 4 : j < 8 ? j : 0;             // sub-block whose top two bits go to bits 6-7
            const int ls_h = __shfl_sync(0xffffffffu, ls, 4 * hi_sub), lm_h = __shfl_sync(0xffffffffu, lm, 4 * hi_sub);
            uint8_t byte;
            if (j < 4) byte = (uint8_t)(ls_a | ((ls_h >> 4) << 6));
            else if (j < 8) byte = (uint8_t)(lm_a | ((lm_h >> 4) << 6));
            else byte = (uint8_t)((ls_a & 0x0F) | ((lm_a & 0x0F) << 4));
            if (lane < 12) o[4 + lane] = byte;
            if (lane == 12) st16(o, d16);
            if (lane == 13) st16(o + 2, m16);
        }
        const float d = half_bits_to_float(d16), dmin = half_bits_to_float(m16);
        const float dd = __fmul_rn(d, (float)ls), dm = __fmul_rn(dmin, (float)lm);
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int q = 0;
            if (dd > 0.0f) q = clampi(round_half_up(__fdiv_rn(__fadd_rn(x[i], dm), dd)), 0, 15);
            packed |= (uint32_t)q << (4 * i);
        }
        // byte l of a 64-weight group = code(l) | code(32 + l) << 4: the even sub-block's lanes
        // take the codes of the odd sub-block's lanes four lanes up
        const uint32_t up = __shfl_down_sync(0xffffffffu, packed, 4);
        if ((sub & 1) == 0) {
            uint32_t w0 = 0, w1 = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                w0 |= (((packed >> (4 * i)) & 0xF) | (((up >> (4 * i)) & 0xF) << 4)) << (8 * i);
                w1 |= (((packed >> (4 * (i + 4))) & 0xF) | (((up >> (4 * (i + 4))) & 0xF) << 4)) << (8 * i);
            }
            *reinterpret_cast<uint2*>(o + 16 + 32 * (sub >> 1) + 8 * (lane & 3)) = make_uint2(w0, w1);
        }
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_quantize(const float* src, void* dst, int64_t n, int kind) {
    if (n == 0) return B200_OK;
    B200_REQUIRE(src && dst && n > 0, "quantize: bad arguments");
    B200_REQUIRE(kind >= 0 && kind <= 4, "quantize: unknown kind %d", kind);
    const int be = kind == 3 ? 256 : 32;
    B200_REQUIRE(n % be == 0, "quantize: n must be a multiple of %d", be);
    B200_REQUIRE((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 7) == 0,
                 "quantize: src must be 16-byte and dst 8-byte aligned");
    const int64_t nb = n / be;
    uint8_t* d = static_cast<uint8_t*>(dst);
    const int64_t warps = kind == 3 ? nb : ceil_div64(nb, 4);
    const unsigned grid = (unsigned)std::min<int64_t>(ceil_div64(warps, 8), (int64_t)num_sms() * 16);
    switch (kind) {
        case 0: quantize32_kernel<0><<<grid, 256, 0, stream()>>>(src, d, nb); break;
        case 1: quantize32_kernel<1><<<grid, 256, 0, stream()>>>(src, d, nb); break;
        case 2: quantize32_kernel<2><<<grid, 256, 0, stream()>>>(src, d, nb); break;
        case 4: quantize32_kernel<4><<<grid, 256, 0, stream()>>>(src, d, nb); break;
        default: quantize_q4k_kernel<<<grid, 256, 0, stream()>>>(src, d, nb); break;
    }
    B200_LAUNCH_CHECK("quantize_kernel");
    return B200_OK;
}
