// Tensor-core dot products of a 16-row weight tile (in shared memory) with up to 8
// activation vectors: the decode-time GEMV mapped onto mma.sync m16n8k16 (weights =
// A, the tokens = the 8 columns of B) so that dequantisation costs about one
// instruction per two weights instead of five per weight.
//
// Numerics.  A holds exact values (Q4_K: the integer nibble, or 16x the nibble for
// the high half, produced with the 0x6400 exponent trick and an exact fp16 subtract;
// fp16 weights as stored).  Each activation is split x = hi + lo into two fp16 values
// (22 significant bits) and both parts are multiplied, accumulation is fp32, and
// the Q4_K sub-block scale and minimum are applied in fp32 afterwards:
//     y += (d*sc) * sum(q*x) - (dmin*m) * sum(x)        per 32-weight sub-block.
// The result differs from the fp32 scalar path only by summation order and by the
// 2^-11 rounding the reference's CPU path applies to each dequantised weight.
#pragma once

#include <cuda_fp16.h>

#include "quant.cuh"

namespace b200 {

#ifdef __CUDACC__
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Activations for the MMA path: per token two fp16 arrays (hi, lo parts) of K values
// and K/32 fp32 sub-block sums.  Token rows are XH_PAD halves longer than K so that
// two tokens' 64-byte segments fall into different bank halves.  Row `zero_row` is
// all zeros and stands in for absent tokens.
constexpr int XH_PAD = 32;
struct XHalf {
    const __half* hi;     // [(tokens+1)][K + XH_PAD]
    const __half* lo;
    const float* sumx;    // [(tokens+1)][K/32]
    int stride;           // K + XH_PAD
    int nsub;             // K / 32
    int zero_row;
};
__host__ __device__ inline size_t xhalf_bytes(int K, int tokens) {
    return (size_t)(tokens + 1) * ((size_t)(K + XH_PAD) * 2 * 2 + (size_t)(K / 32) * 4);
}

// Position of activation k inside its token row.  Q4_K: within every aligned run of 8
// the order is 0,2,1,3,4,6,5,7 so that one 16-byte load yields the four B registers
// of the two MMAs that consume one 32-bit word of nibbles.
template <int KIND>
__device__ __forceinline__ int xh_index(int k) {
    if (KIND == 3) {
        const int r = k & 7;
        const int p = (r & 4) | ((r & 1) << 1) | ((r >> 1) & 1);
        return (k & ~7) | p;
    }
    return k;
}

__device__ __forceinline__ uint32_t nib_lo(uint32_t w) {   // nibbles at bits 0-3 and 16-19 -> half2 (q, q)
    const uint32_t t = (w & 0x000F000Fu) | 0x64006400u;
    const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&t), __half2half2(__ushort_as_half(0x6400)));
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t nib_hi(uint32_t w) {   // nibbles at bits 4-7 and 20-23 -> half2 (16q, 16q)
    const uint32_t t = (w & 0x00F000F0u) | 0x64006400u;
    const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&t), __half2half2(__ushort_as_half(0x6400)));
    return *reinterpret_cast<const uint32_t*>(&h);
}

// 32-bit shared-memory loads (tiles and staged activations live in shared memory; plain
// pointers would carry 64-bit generic address arithmetic through the loop).
__device__ __forceinline__ uint4 lds_u4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds_u2(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t a) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
    return v;
}

// Q4_K: partial sums over this warp's share of K - the 64-weight groups
// [part * per, (part + 1) * per), per = ceil(K / 64 / nparts) - for the 16 rows at `tile`
// (row stride rb bytes; tile and xh in shared memory).  acc: the m16n8 accumulator fragment
// (rows lane/4 and lane/4+8, columns = tokens 2*(lane%4), +1).  A super-block's header is
// decoded once for the groups of the range that share it.
__device__ __forceinline__ void tile_dot_q4k(const uint8_t* tile, int rb, int K, const XHalf& xh, int M, int part,
                                             int nparts, int lane, float (&acc)[4]) {
    const int gid = lane >> 2, tig = lane & 3;
    const int tok = gid < M ? gid : xh.zero_row;
    const int c0 = 2 * tig, c1 = c0 + 1;
    const int groups = K >> 6;
    const int per = (groups + nparts - 1) / nparts;
    const int g0 = part * per, g1 = min(groups, g0 + per);
    const int row = lane & 15, hi = lane >> 4;
    const uint32_t tile_s = static_cast<uint32_t>(__cvta_generic_to_shared(tile));
    const uint32_t hdr_a = tile_s + row * rb;
    const uint32_t wa_a = tile_s + gid * rb + 16 + 8 * tig;
    const uint32_t wb_a = wa_a + 8 * rb;
    const uint32_t x_off = (uint32_t)(tok * xh.stride + 8 * tig) * 2 + g0 * 128;
    uint32_t xh_a = static_cast<uint32_t>(__cvta_generic_to_shared(xh.hi)) + x_off;
    uint32_t xl_a = static_cast<uint32_t>(__cvta_generic_to_shared(xh.lo)) + x_off;
    const uint32_t sum_s = static_cast<uint32_t>(__cvta_generic_to_shared(xh.sumx));
    uint32_t s0_a = sum_s + (uint32_t)((c0 < M ? c0 : xh.zero_row) * xh.nsub) * 4 + g0 * 8;
    uint32_t s1_a = sum_s + (uint32_t)((c1 < M ? c1 : xh.zero_row) * xh.nsub) * 4 + g0 * 8;
    uint32_t sc_lo = 0, sc_hi = 0, mn_lo = 0, mn_hi = 0;
    float d = 0.0f, dmin = 0.0f;
    int cur_sb = -1;
    for (int g = g0; g < g1; ++g, xh_a += 128, xl_a += 128, s0_a += 8, s1_a += 8) {
        const int sb = g >> 2, j = g & 3;
        if (sb != cur_sb) {                       // uniform over the warp
            cur_sb = sb;
            // this lane's row: d, dmin and the eight 6-bit (scale, min) pairs as bytes of two words each
            const uint4 h4 = lds_u4(hdr_a + sb * 144);
            d = half_bits_to_float((uint16_t)(h4.x & 0xFFFF));
            dmin = half_bits_to_float((uint16_t)(h4.x >> 16));
            sc_lo = h4.y & 0x3F3F3F3Fu;
            mn_lo = h4.z & 0x3F3F3F3Fu;
            sc_hi = (h4.w & 0x0F0F0F0Fu) | ((h4.y >> 2) & 0x30303030u);
            mn_hi = ((h4.w >> 4) & 0x0F0F0F0Fu) | ((h4.z >> 2) & 0x30303030u);
        }
        // this lane's (row, sub-block 2 j + hi) scale pair; shared with the warp by shuffles
        const uint32_t sel = 2 * j + hi;
        const float P = d * (float)(__byte_perm(sc_lo, sc_hi, sel) & 0xFFu) * (hi ? 0.0625f : 1.0f);
        const float Q = dmin * (float)(__byte_perm(mn_lo, mn_hi, sel) & 0xFFu);
        const float P_lo_a = __shfl_sync(0xffffffffu, P, gid), P_lo_b = __shfl_sync(0xffffffffu, P, gid + 8);
        const float P_hi_a = __shfl_sync(0xffffffffu, P, 16 + gid), P_hi_b = __shfl_sync(0xffffffffu, P, 24 + gid);
        const float Q_lo_a = __shfl_sync(0xffffffffu, Q, gid), Q_lo_b = __shfl_sync(0xffffffffu, Q, gid + 8);
        const float Q_hi_a = __shfl_sync(0xffffffffu, Q, 16 + gid), Q_hi_b = __shfl_sync(0xffffffffu, Q, 24 + gid);
        const uint32_t woff = sb * 144 + 32 * j;
        const uint2 wa = lds_u2(wa_a + woff);
        const uint2 wb = lds_u2(wb_a + woff);
        const uint4 bh_lo = lds_u4(xh_a), bl_lo = lds_u4(xl_a), bh_hi = lds_u4(xh_a + 64), bl_hi = lds_u4(xl_a + 64);
        float cl[4] = {0.f, 0.f, 0.f, 0.f}, ch[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const uint32_t a0 = nib_lo(wa.x), a1 = nib_lo(wb.x), a2 = nib_lo(wa.x >> 8), a3 = nib_lo(wb.x >> 8);
            mma_16816(cl, a0, a1, a2, a3, bh_lo.x, bh_lo.y);
            mma_16816(cl, a0, a1, a2, a3, bl_lo.x, bl_lo.y);
            const uint32_t e0 = nib_hi(wa.x), e1 = nib_hi(wb.x), e2 = nib_hi(wa.x >> 8), e3 = nib_hi(wb.x >> 8);
            mma_16816(ch, e0, e1, e2, e3, bh_hi.x, bh_hi.y);
            mma_16816(ch, e0, e1, e2, e3, bl_hi.x, bl_hi.y);
        }
        {
            const uint32_t a0 = nib_lo(wa.y), a1 = nib_lo(wb.y), a2 = nib_lo(wa.y >> 8), a3 = nib_lo(wb.y >> 8);
            mma_16816(cl, a0, a1, a2, a3, bh_lo.z, bh_lo.w);
            mma_16816(cl, a0, a1, a2, a3, bl_lo.z, bl_lo.w);
            const uint32_t e0 = nib_hi(wa.y), e1 = nib_hi(wb.y), e2 = nib_hi(wa.y >> 8), e3 = nib_hi(wb.y >> 8);
            mma_16816(ch, e0, e1, e2, e3, bh_hi.z, bh_hi.w);
            mma_16816(ch, e0, e1, e2, e3, bl_hi.z, bl_hi.w);
        }
        const float2 s0 = lds_f2(s0_a), s1 = lds_f2(s1_a);
        acc[0] += P_lo_a * cl[0] - Q_lo_a * s0.x + P_hi_a * ch[0] - Q_hi_a * s0.y;
        acc[1] += P_lo_a * cl[1] - Q_lo_a * s1.x + P_hi_a * ch[1] - Q_hi_a * s1.y;
        acc[2] += P_lo_b * cl[2] - Q_lo_b * s0.x + P_hi_b * ch[2] - Q_hi_b * s0.y;
        acc[3] += P_lo_b * cl[3] - Q_lo_b * s1.x + P_hi_b * ch[3] - Q_hi_b * s1.y;
    }
}

// fp16 weights: 32-wide k chunks c = part, part + nparts, ...
__device__ __forceinline__ void tile_dot_f16(const uint8_t* tile, int rb, int K, const XHalf& xh, int M, int part,
                                             int nparts, int lane, float (&acc)[4]) {
    const int gid = lane >> 2, tig = lane & 3;
    const int tok = gid < M ? gid : xh.zero_row;
    const __half* xh_row = xh.hi + (size_t)tok * xh.stride;
    const __half* xl_row = xh.lo + (size_t)tok * xh.stride;
    const int chunks = K >> 5;
    for (int c = part; c < chunks; c += nparts) {
        const int k0 = 32 * c + 8 * tig;
        const uint4 ra = *reinterpret_cast<const uint4*>(tile + (size_t)gid * rb + (size_t)k0 * 2);
        const uint4 rb8 = *reinterpret_cast<const uint4*>(tile + (size_t)(gid + 8) * rb + (size_t)k0 * 2);
        const uint4 bh = *reinterpret_cast<const uint4*>(xh_row + k0);
        const uint4 bl = *reinterpret_cast<const uint4*>(xl_row + k0);
        mma_16816(acc, ra.x, rb8.x, ra.y, rb8.y, bh.x, bh.y);
        mma_16816(acc, ra.x, rb8.x, ra.y, rb8.y, bl.x, bl.y);
        mma_16816(acc, ra.z, rb8.z, ra.w, rb8.w, bh.z, bh.w);
        mma_16816(acc, ra.z, rb8.z, ra.w, rb8.w, bl.z, bl.w);
    }
}
#endif

}  // namespace b200
