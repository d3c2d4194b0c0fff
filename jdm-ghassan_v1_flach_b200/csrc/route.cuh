// Router tail shared by the few-token and the many-token MoE kernels.
#pragma once

#include "common.cuh"

namespace b200 {

#ifdef __CUDACC__
// One warp: softmax over ne logits, K rounds of arg-max (value descending, index
// ascending, candidates must exceed -1e30), renormalised mixture weights -
// core/math_cpu.cpp:546-558 and core/moe_cpu.cpp:85-98,233-254 bit for bit except
// exp(), evaluated in double and rounded.  s_p / s_sel: ne floats of scratch.
__device__ __forceinline__ void route_finish_warp(const float* __restrict__ logits, const float* __restrict__ bias,
                                                  int ne, int K, float* s_p, float* s_sel, int* s_idx, float* s_w,
                                                  float* probs_out, int lane) {
    float mx = __ldcg(logits);   // L2 loads: another CTA of the same kernel may have written the logits
    for (int e = lane; e < ne; e += 32) mx = fmaxf(mx, __ldcg(logits + e));
    mx = warp_max(mx);
    for (int e = lane; e < ne; e += 32) s_p[e] = (float)exp((double)__fsub_rn(__ldcg(logits + e), mx));
    __syncwarp();
    float inv = 0.0f;
    if (lane == 0) {
        float sum = 0.0f;
        for (int e = 0; e < ne; ++e) sum = __fadd_rn(sum, s_p[e]);
        inv = (sum > 1e-12f) ? __fdiv_rn(1.0f, sum) : 0.0f;
    }
    inv = __shfl_sync(0xffffffffu, inv, 0);
    for (int e = lane; e < ne; e += 32) {
        const float pr = __fmul_rn(s_p[e], inv);
        s_p[e] = pr;
        s_sel[e] = bias ? __fadd_rn(pr, bias[e]) : pr;
        if (probs_out) probs_out[e] = pr;
    }
    __syncwarp();
    for (int k = 0; k < K; ++k) {
        float bv = -1e30f;
        int bi = -1;
        for (int e = lane; e < ne; e += 32) {
            bool taken = false;
            for (int j = 0; j < k; ++j) taken |= (s_idx[j] == e);
            const float v = s_sel[e];
            if (!taken && v > bv) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        if (lane == 0) s_idx[k] = bi < 0 ? 0 : bi;
        __syncwarp();
    }
    if (lane == 0) {
        float sum_w = 0.0f;
        for (int k = 0; k < K; ++k) { s_w[k] = s_p[s_idx[k]]; sum_w = __fadd_rn(sum_w, s_w[k]); }
        if (sum_w > 1e-8f) {
            const float inv_w = __fdiv_rn(1.0f, sum_w);
            for (int k = 0; k < K; ++k) s_w[k] = __fmul_rn(s_w[k], inv_w);
        } else {
            const float uni = __fdiv_rn(1.0f, (float)K);
            for (int k = 0; k < K; ++k) s_w[k] = uni;
        }
    }
    __syncwarp();
}
#endif

}  // namespace b200
