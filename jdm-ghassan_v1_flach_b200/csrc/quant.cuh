// Device-side readers of the packed weight formats.
//
// kind 0 = Q4_0 (18 B / 32 weights), 1 = Q4_1 (20 B / 32), 2 = Q8_0 (34 B / 32):
// the reference engine's blocks (core/dtype.h:35-53); values follow its CPU
// dequantiser (core/ops.cpp:313-334): Q4_0 (nib-8)*d, Q4_1 nib*d+m, Q8_0 q*d, low
// nibble = element j, high nibble = element j+16, d and m fp16.  kind 3 = Q4_K
// (144 B / 256 weights, public GGML layout: f16 d, f16 dmin, 12 B of 6-bit
// scales/mins, 128 B of nibbles; 64 weights share 32 bytes, low nibbles first).
//
// Every value is produced with explicit round-to-nearest single operations
// (__fmul_rn/__fadd_rn, never a fused multiply-add) so that the bits equal the CPU
// path's, which is compiled without FMA contraction.
#pragma once

#include "common.cuh"

namespace b200 {

__host__ __device__ constexpr int q_block_elems(int kind) { return kind == 3 ? 256 : 32; }
__host__ __device__ constexpr int q_block_bytes(int kind) {
    return kind == 0 ? 18 : kind == 1 ? 20 : kind == 2 ? 34 : 144;
}
// Bytes of one packed row of K weights (K is a multiple of the block size).
__host__ __device__ inline int64_t q_row_bytes(int kind, int K) {
    return (int64_t)(K / q_block_elems(kind)) * q_block_bytes(kind);
}

#ifdef __CUDACC__
__device__ __forceinline__ float ld_half(const uint8_t* p) {
    return half_bits_to_float(*reinterpret_cast<const uint16_t*>(p));
}

// The value the reference's CPU inference path multiplies with: fp16(v) widened.
__device__ __forceinline__ float round_through_half(float v) {
    return __half2float(__float2half_rn(v));
}

// 6-bit (scale, min) pair j of a Q4_K super-block; sc points at the 12 bytes.
__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t* sc, int& s, int& m) {
    if (j < 4) {
        s = sc[j] & 63;
        m = sc[j + 4] & 63;
    } else {
        s = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4);
        m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
    }
}

// The same from the three 32-bit words that hold the 12 bytes (bytes 4..15 of the
// super-block: y, z, w of a 16-byte header load): shifts and selects only, so a header
// held in registers is never spilled to be indexed bytewise.
__device__ __forceinline__ void q4k_scale_min_regs(int j, uint32_t y, uint32_t z, uint32_t w, int& s, int& m) {
    const int sh = 8 * (j & 3);
    const uint32_t by = (y >> sh) & 0xFFu, bz = (z >> sh) & 0xFFu, bw = (w >> sh) & 0xFFu;
    if (j < 4) {
        s = (int)(by & 63u);
        m = (int)(bz & 63u);
    } else {
        s = (int)((bw & 0x0Fu) | ((by >> 6) << 4));
        m = (int)((bw >> 4) | ((bz >> 6) << 4));
    }
}

// One weight by flat index i, exact fp32 (used by the materialising dequantiser
// and by slow general paths).
template <int KIND>
__device__ __forceinline__ float q_value(const uint8_t* base, int64_t i) {
    if (KIND == 3) {
        const uint8_t* blk = base + (i >> 8) * 144;
        const int r = (int)(i & 255), grp = r >> 6, hi = (r >> 5) & 1, l = r & 31;
        int s, m;
        q4k_scale_min(2 * grp + hi, blk + 4, s, m);
        const float d1 = __fmul_rn(ld_half(blk), (float)s);
        const float m1 = __fmul_rn(ld_half(blk + 2), (float)m);
        const uint8_t byte = blk[16 + 32 * grp + l];
        const int q = hi ? (byte >> 4) : (byte & 0x0F);
        return __fsub_rn(__fmul_rn(d1, (float)q), m1);
    }
    const int64_t b = i >> 5;
    const int j = (int)(i & 31);
    if (KIND == 0) {
        const uint8_t* blk = base + b * 18;
        const uint8_t byte = blk[2 + (j & 15)];
        const int q = (j < 16) ? (byte & 0x0F) : (byte >> 4);
        return __fmul_rn((float)(q - 8), ld_half(blk));
    }
    if (KIND == 1) {
        const uint8_t* blk = base + b * 20;
        const uint8_t byte = blk[4 + (j & 15)];
        const int q = (j < 16) ? (byte & 0x0F) : (byte >> 4);
        return __fadd_rn(__fmul_rn((float)q, ld_half(blk)), ld_half(blk + 2));
    }
    const uint8_t* blk = base + b * 34;
    return __fmul_rn((float)reinterpret_cast<const int8_t*>(blk + 2)[j], ld_half(blk));
}

// ---- 32-weight units -------------------------------------------------------
// The GEMV kernels walk a packed row in units of 32 weights held in registers.
// For the 32-element formats a unit is one block (weights k0..k0+31).  For Q4_K a
// unit is one 16-byte slice of the nibble area: 16 low nibbles (weights
// k0..k0+15) and 16 high nibbles (weights k0+32..k0+47).  unit_k() gives the two
// 16-weight runs' first k.
template <int KIND>
__device__ __forceinline__ int units_per_row(int K) { return K / 32; }

template <int KIND>
__device__ __forceinline__ void unit_k(int u, int& k_lo, int& k_hi) {
    if (KIND == 3) {
        const int sb = u >> 3, c = u & 7;
        k_lo = sb * 256 + (c >> 1) * 64 + (c & 1) * 16;
        k_hi = k_lo + 32;
    } else {
        k_lo = u * 32;
        k_hi = k_lo + 16;
    }
}

// Dequantise unit u of the packed row into w[0..15] (first run) and w[16..31]
// (second run).  ROUND16: round each value through fp16 like the reference's CPU
// inference path does.
template <int KIND, bool ROUND16>
__device__ __forceinline__ void load_unit(const uint8_t* row, int u, float (&w)[32]) {
    if (KIND == 3) {
        const uint8_t* blk = row + (u >> 3) * 144;
        const int c = u & 7, grp = c >> 1;
        const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
        const uint4 qs = *reinterpret_cast<const uint4*>(blk + 16 + 16 * c);
        int s0, m0, s1, m1;
        q4k_scale_min_regs(2 * grp, hdr.y, hdr.z, hdr.w, s0, m0);
        q4k_scale_min_regs(2 * grp + 1, hdr.y, hdr.z, hdr.w, s1, m1);
        const float d = half_bits_to_float((uint16_t)(hdr.x & 0xFFFF));
        const float dmin = half_bits_to_float((uint16_t)(hdr.x >> 16));
        const float d_lo = __fmul_rn(d, (float)s0), d_hi = __fmul_rn(d, (float)s1);
        const float m_lo = __fmul_rn(dmin, (float)m0), m_hi = __fmul_rn(dmin, (float)m1);
        const uint32_t words[4] = {qs.x, qs.y, qs.z, qs.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t byte = (words[i >> 2] >> (8 * (i & 3))) & 0xFF;
            float lo = __fsub_rn(__fmul_rn(d_lo, (float)(byte & 0x0F)), m_lo);
            float hi = __fsub_rn(__fmul_rn(d_hi, (float)(byte >> 4)), m_hi);
            w[i] = ROUND16 ? round_through_half(lo) : lo;
            w[16 + i] = ROUND16 ? round_through_half(hi) : hi;
        }
        return;
    }
    if (KIND == 2) {
        const uint16_t* blk = reinterpret_cast<const uint16_t*>(row + (int64_t)u * 34);
        const float d = half_bits_to_float(blk[0]);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint16_t pair = blk[1 + i];
            const float a = __fmul_rn((float)(int8_t)(pair & 0xFF), d);
            const float b = __fmul_rn((float)(int8_t)(pair >> 8), d);
            w[2 * i] = ROUND16 ? round_through_half(a) : a;
            w[2 * i + 1] = ROUND16 ? round_through_half(b) : b;
        }
        return;
    }
    // Q4_0 / Q4_1: 2-byte aligned blocks, 16 nibble bytes
    const int bb = KIND == 0 ? 18 : 20;
    const uint16_t* blk = reinterpret_cast<const uint16_t*>(row + (int64_t)u * bb);
    const float d = half_bits_to_float(blk[0]);
    const float mn = KIND == 1 ? half_bits_to_float(blk[1]) : 0.0f;
    const uint16_t* qs = blk + (KIND == 0 ? 1 : 2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint16_t pair = qs[i];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int byte = (pair >> (8 * h)) & 0xFF;
            float lo, hi;
            if (KIND == 0) {
                lo = __fmul_rn((float)((byte & 0x0F) - 8), d);
                hi = __fmul_rn((float)((byte >> 4) - 8), d);
            } else {
                lo = __fadd_rn(__fmul_rn((float)(byte & 0x0F), d), mn);
                hi = __fadd_rn(__fmul_rn((float)(byte >> 4), d), mn);
            }
            w[2 * i + h] = ROUND16 ? round_through_half(lo) : lo;
            w[16 + 2 * i + h] = ROUND16 ? round_through_half(hi) : hi;
        }
    }
}
#endif

}  // namespace b200
