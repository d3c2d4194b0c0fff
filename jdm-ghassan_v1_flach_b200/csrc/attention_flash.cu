// Prefill attention for long sequences: causal (optionally windowed / segment-masked)
// softmax(q k^T) v without ever forming the [T, T] score matrix, on tensor cores.
//
// Same result as attn_prefill_kernel (attention.cu) and as cpu::attention_forward_ex
// (core/attn_cpu.cpp:29-94) up to fp16 rounding of q, k, v and of the probabilities
// (accumulation and the softmax statistics are fp32) - the reference's CUDA path feeds
// its batched cuBLAS GEMMs fp16 copies as well (cuda/attention.cu:432-499).
//
// One CTA = 128 queries of one (sequence, head); each of its 8 warps owns 16 query rows
// (a key / value tile staged once serves 128 queries; a warp skips the tiles that lie
// entirely above its rows' diagonal).
// Keys and values arrive 64 at a time through shared memory (both row-major fp16, rows
// padded by 16 bytes so that the eight row addresses of an ldmatrix tile fall into
// different bank groups); K fragments come from plain ldmatrix loads, V fragments from
// transposing ones.  Scores and outputs live in mma.sync.m16n8k16 accumulator fragments,
// and the score fragment of a 16-key slice is reused directly as the A operand of the
// probability-times-value product.
#include <cuda_fp16.h>

#include "mma_tile.cuh"

namespace b200 {

constexpr int FA_BM = 128, FA_BN = 64, FA_THREADS = 256;

__device__ __forceinline__ void fa_ldsm_x4(uint32_t (&r)[4], const __half* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void fa_ldsm_x4_t(uint32_t (&r)[4], const __half* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(p)));
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int HD>
__global__ void __launch_bounds__(FA_THREADS)
attn_flash_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  float* __restrict__ out, int T, int H, int KV, float scale, int window,
                  const int32_t* __restrict__ seg) {
    constexpr int LDK = HD + 8;
    __shared__ __align__(16) __half Ks[FA_BN * LDK];
    __shared__ __align__(16) __half Vs[FA_BN * LDK];
    __shared__ int32_t s_seg[FA_BN];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int lj = lane >> 3, lr = lane & 7;                // ldmatrix: which 8 x 8 tile, which of its rows
    // query tiles are handed out last first: under the causal mask a tile's work grows with
    // its position, and the heavy ones should not be what the last wave is made of
    const int q0 = (gridDim.x - 1 - blockIdx.x) * FA_BM, h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (H / KV);
    const int64_t qs = (int64_t)T * H * HD, kvs = (int64_t)T * KV * HD;
    const float* qb = q + b * qs + (int64_t)h * HD;
    const float* kb = k + b * kvs + (int64_t)kvh * HD;
    const float* vb = v + b * kvs + (int64_t)kvh * HD;
    const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;        // this lane's two query rows
    const float qscale = scale * 1.44269504088896f;         // scores in log2 units: p = 2^(s - m)

    // query fragments (pre-scaled), rows past T read as zero
    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        const int c = ks * 16 + 2 * t4;
        float2 x0 = make_float2(0.f, 0.f), x1 = x0, x2 = x0, x3 = x0;
        if (r0 < T) {
            x0 = *reinterpret_cast<const float2*>(qb + (int64_t)r0 * H * HD + c);
            x2 = *reinterpret_cast<const float2*>(qb + (int64_t)r0 * H * HD + c + 8);
        }
        if (r1 < T) {
            x1 = *reinterpret_cast<const float2*>(qb + (int64_t)r1 * H * HD + c);
            x3 = *reinterpret_cast<const float2*>(qb + (int64_t)r1 * H * HD + c + 8);
        }
        qa[ks][0] = pack_half2(x0.x * qscale, x0.y * qscale);
        qa[ks][1] = pack_half2(x1.x * qscale, x1.y * qscale);
        qa[ks][2] = pack_half2(x2.x * qscale, x2.y * qscale);
        qa[ks][3] = pack_half2(x3.x * qscale, x3.y * qscale);
    }
    const int32_t seg0 = (seg && r0 < T) ? seg[(int64_t)b * T + r0] : -1;
    const int32_t seg1 = (seg && r1 < T) ? seg[(int64_t)b * T + r1] : -1;
    const int lo0 = window > 0 ? max(0, r0 - window + 1) : 0, lo1 = window > 0 ? max(0, r1 - window + 1) : 0;

    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;

    const int q_last = min(T - 1, q0 + FA_BM - 1);
    const int j_first = window > 0 ? max(0, q0 - window + 1) : 0;
    for (int kv0 = (j_first / FA_BN) * FA_BN; kv0 <= q_last; kv0 += FA_BN) {
        __syncthreads();                                    // the previous tile has been consumed
        for (int i = threadIdx.x; i < FA_BN * (HD / 4); i += FA_THREADS) {
            const int key = i / (HD / 4), c = (i - key * (HD / 4)) * 4;
            float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), vv = kk;
            if (kv0 + key < T) {
                kk = *reinterpret_cast<const float4*>(kb + (int64_t)(kv0 + key) * KV * HD + c);
                vv = *reinterpret_cast<const float4*>(vb + (int64_t)(kv0 + key) * KV * HD + c);
            }
            *reinterpret_cast<uint2*>(&Ks[key * LDK + c]) = make_uint2(pack_half2(kk.x, kk.y), pack_half2(kk.z, kk.w));
            *reinterpret_cast<uint2*>(&Vs[key * LDK + c]) = make_uint2(pack_half2(vv.x, vv.y), pack_half2(vv.z, vv.w));
        }
        if (threadIdx.x < FA_BN) s_seg[threadIdx.x] = (seg && kv0 + threadIdx.x < T) ? seg[(int64_t)b * T + kv0 + threadIdx.x] : 0;
        __syncthreads();

        // tiles entirely in this warp's future (or before its window) contribute nothing
        const int w_first = q0 + warp * 16, w_last = w_first + 15;
        if (kv0 > w_last || (window > 0 && kv0 + FA_BN - 1 < w_first - window + 1)) continue;
        // scores of this warp's 16 rows against the 64 keys
        float s[FA_BN / 8][4];
#pragma unroll
        for (int np = 0; np < FA_BN / 16; ++np) {           // two 8-key tiles per ldmatrix
            s[2 * np][0] = s[2 * np][1] = s[2 * np][2] = s[2 * np][3] = 0.0f;
            s[2 * np + 1][0] = s[2 * np + 1][1] = s[2 * np + 1][2] = s[2 * np + 1][3] = 0.0f;
            // tiles: (keys +0..7, k 0..7) (keys +0..7, k 8..15) (keys +8..15, k 0..7) (keys +8..15, k 8..15)
            const __half* kp = &Ks[(np * 16 + (lj >> 1) * 8 + lr) * LDK + (lj & 1) * 8];
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                uint32_t kb[4];
                fa_ldsm_x4(kb, kp + ks * 16);
                mma_16816(s[2 * np], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[0], kb[1]);
                mma_16816(s[2 * np + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[2], kb[3]);
            }
        }
        // mask, running maximum
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int nt = 0; nt < FA_BN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int kl = nt * 8 + 2 * t4 + e, j = kv0 + kl;
                const int32_t sj = s_seg[kl];
                const bool ok0 = j <= r0 && j >= lo0 && r0 < T && !(seg && seg0 >= 0 && sj != seg0);
                const bool ok1 = j <= r1 && j >= lo1 && r1 < T && !(seg && seg1 >= 0 && sj != seg1);
                s[nt][e] = ok0 ? s[nt][e] : -INFINITY;
                s[nt][2 + e] = ok1 ? s[nt][2 + e] : -INFINITY;
                mx0 = fmaxf(mx0, s[nt][e]);
                mx1 = fmaxf(mx1, s[nt][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        // rows with nothing visible yet keep a finite reference so that 2^(-inf - ref) = 0
        const float ref0 = mx0 == -INFINITY ? 0.0f : mx0, ref1 = mx1 == -INFINITY ? 0.0f : mx1;
        const float al0 = exp2f(m0 - ref0), al1 = exp2f(m1 - ref1);   // m = -inf -> 0
        m0 = mx0;
        m1 = mx1;
        l0 *= al0;
        l1 *= al1;
#pragma unroll
        for (int d = 0; d < HD / 8; ++d) {
            o[d][0] *= al0; o[d][1] *= al0;
            o[d][2] *= al1; o[d][3] *= al1;
        }
        // probabilities -> A fragments; P V
#pragma unroll
        for (int kk = 0; kk < FA_BN / 16; ++kk) {
            float p[2][4];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                p[u][0] = exp2f(s[2 * kk + u][0] - ref0);
                p[u][1] = exp2f(s[2 * kk + u][1] - ref0);
                p[u][2] = exp2f(s[2 * kk + u][2] - ref1);
                p[u][3] = exp2f(s[2 * kk + u][3] - ref1);
                l0 += p[u][0] + p[u][1];
                l1 += p[u][2] + p[u][3];
            }
            const uint32_t a0 = pack_half2(p[0][0], p[0][1]), a1 = pack_half2(p[0][2], p[0][3]);
            const uint32_t a2 = pack_half2(p[1][0], p[1][1]), a3 = pack_half2(p[1][2], p[1][3]);
            // V tiles of this 16-key slice: (keys 0..7, d +0..7) (keys 8..15, d +0..7) (keys 0..7, d +8..15) ...
            const __half* vp = &Vs[(kk * 16 + (lj & 1) * 8 + lr) * LDK + (lj >> 1) * 8];
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
                uint32_t vb[4];
                fa_ldsm_x4_t(vb, vp + dp * 16);
                mma_16816(o[2 * dp], a0, a1, a2, a3, vb[0], vb[1]);
                mma_16816(o[2 * dp + 1], a0, a1, a2, a3, vb[2], vb[3]);
            }
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, inv1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
    float* ob = out + b * qs + (int64_t)h * HD;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) {
        const int c = d * 8 + 2 * t4;
        if (r0 < T) *reinterpret_cast<float2*>(ob + (int64_t)r0 * H * HD + c) = make_float2(o[d][0] * inv0, o[d][1] * inv0);
        if (r1 < T) *reinterpret_cast<float2*>(ob + (int64_t)r1 * H * HD + c) = make_float2(o[d][2] * inv1, o[d][3] * inv1);
    }
}

// Returns B200_EUNSUPPORTED for head sizes it has no instance for.
int attention_flash(const float* q, const float* k, const float* v, float* out, int B, int T, int H, int KV, int hd,
                    float scale, int window, const int32_t* seg) {
    const dim3 grid(ceil_div(T, FA_BM), H, B);
    if (hd == 128) attn_flash_kernel<128><<<grid, FA_THREADS, 0, stream()>>>(q, k, v, out, T, H, KV, scale, window, seg);
    else if (hd == 64) attn_flash_kernel<64><<<grid, FA_THREADS, 0, stream()>>>(q, k, v, out, T, H, KV, scale, window, seg);
    else return fail(B200_EUNSUPPORTED, "attention_flash: head_dim %d", hd);
    B200_LAUNCH_CHECK("attn_flash_kernel");
    return B200_OK;
}

}  // namespace b200
