// GQA attention: single-token decode over a ring or paged KV cache (split-KV,
// one pass over K/V for all query heads of a KV group) and causal prefill.
//
// Reference arithmetic: core/attn_cpu.cpp:29-94 (prefill, window, segment mask),
// :151-254 (ring decode, fp32 and fp16 caches); kernels replaced:
// cuda/attention.cu:317-499 and :614-809.
//
// s_j = scale * q_h . k_j ; p = softmax_j(s) ; o = sum_j p_j v_j, computed with a
// running (max, sum) per query head so no [H, len] score buffer is needed; the
// caller's `scratch` argument is accepted and unused.
#include <algorithm>

#include <mutex>

#include "common.cuh"

namespace b200 {

constexpr int ATT_WARPS = 4;
constexpr int ATT_GMAX = 8;     // query heads of one KV group handled per block

// Where the key/value row of logical position j lives.
struct KvLocator {
    // ring (single sequence): pinned prefix + rolling window (core/attn_cpu.cpp:151-156)
    int ring_start, pinned, ring_cap;
    // paged (batched): page table row of this sequence
    const int32_t* pages;
    int page;
    __device__ __forceinline__ int64_t row(int j, bool paged) const {
        if (paged) return (int64_t)pages[j / page] * page + (j % page);
        if (j < pinned) return j;
        return (int64_t)pinned + (ring_start + (j - pinned)) % ring_cap;
    }
};

template <int EPL, bool HALF>
__device__ __forceinline__ void load_row(const void* base, int64_t elem_off, int lane, float (&v)[EPL]) {
    if (HALF) {
        const uint16_t* p = static_cast<const uint16_t*>(base) + elem_off + lane * EPL;
        if (EPL == 8) {
            const uint4 u = *reinterpret_cast<const uint4*>(p);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                v[2 * i] = f.x; v[2 * i + 1] = f.y;
            }
        } else if (EPL == 4) {
            const uint2 u = *reinterpret_cast<const uint2*>(p);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
            v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
        } else if (EPL == 2) {
            const uint32_t u = *reinterpret_cast<const uint32_t*>(p);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u));
            v[0] = a.x; v[1] = a.y;
        } else {
            v[0] = half_bits_to_float(p[0]);
        }
    } else {
        const float* p = static_cast<const float*>(base) + elem_off + lane * EPL;
#pragma unroll
        for (int i = 0; i < EPL; ++i) v[i] = p[i];
    }
}

struct DecodeArgs {
    const float* q;        // [batch, H, hd]
    const void* kc;
    const void* vc;        // [rows, KV*hd]
    float* part;           // [batch, H, splits, hd + 2]  (o, m, l)
    const int32_t* page_table;   // [batch, max_pages] or null
    const int32_t* seq_lens;     // [batch] or null
    int H, KV, hd, group, splits, chunk;
    int cur_len, j0;       // ring mode
    int ring_start, pinned, ring_cap;
    int max_pages, page;
    float scale;
};

// grid (splits, KV * ceil(group / GMAX), batch)
template <int EPL, bool HALF, bool PAGED>
__global__ void __launch_bounds__(ATT_WARPS * 32) attn_decode_split_kernel(DecodeArgs a) {
    __shared__ float sm_o[ATT_WARPS][ATT_GMAX][EPL * 32];
    __shared__ float sm_ml[ATT_WARPS][ATT_GMAX][2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gblocks = (a.group + ATT_GMAX - 1) / ATT_GMAX;
    const int kvh = blockIdx.y / gblocks, gb = blockIdx.y % gblocks;
    const int b = blockIdx.z;
    const int g0 = gb * ATT_GMAX;
    const int G = min(ATT_GMAX, a.group - g0);
    const int len = PAGED ? a.seq_lens[b] : a.cur_len;
    const int jbeg = (PAGED ? 0 : a.j0) + blockIdx.x * a.chunk;
    const int jend = min(len, jbeg + a.chunk);
    KvLocator loc;
    loc.ring_start = a.ring_start; loc.pinned = a.pinned; loc.ring_cap = a.ring_cap;
    loc.pages = PAGED ? a.page_table + (int64_t)b * a.max_pages : nullptr;
    loc.page = a.page;

    float q[ATT_GMAX][EPL], o[ATT_GMAX][EPL], m[ATT_GMAX], l[ATT_GMAX];
#pragma unroll
    for (int g = 0; g < ATT_GMAX; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) o[g][i] = 0.0f;
        if (g < G) {
            const int h = kvh * a.group + g0 + g;
            load_row<EPL, false>(a.q, ((int64_t)b * a.H + h) * a.hd, lane, q[g]);
        } else {
#pragma unroll
            for (int i = 0; i < EPL; ++i) q[g][i] = 0.0f;
        }
    }
    const int kv_stride = a.KV * a.hd;
    for (int j = jbeg + warp; j < jend; j += ATT_WARPS) {
        const int64_t off = loc.row(j, PAGED) * kv_stride + (int64_t)kvh * a.hd;
        float kv[EPL], vv[EPL];
        load_row<EPL, HALF>(a.kc, off, lane, kv);
        load_row<EPL, HALF>(a.vc, off, lane, vv);
#pragma unroll
        for (int g = 0; g < ATT_GMAX; ++g) {
            if (g < G) {
                float s = 0.0f;
#pragma unroll
                for (int i = 0; i < EPL; ++i) s += q[g][i] * kv[i];
                s = warp_sum(s) * a.scale;
                const float mn = fmaxf(m[g], s);
                const float corr = expf(m[g] - mn);     // exp(-inf) = 0 on the first key
                const float p = expf(s - mn);
                l[g] = l[g] * corr + p;
#pragma unroll
                for (int i = 0; i < EPL; ++i) o[g][i] = o[g][i] * corr + p * vv[i];
                m[g] = mn;
            }
        }
    }
    // combine the warps of this block
#pragma unroll
    for (int g = 0; g < ATT_GMAX; ++g) {
        if (g < G) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) sm_o[warp][g][lane * EPL + i] = o[g][i];
            if (lane == 0) { sm_ml[warp][g][0] = m[g]; sm_ml[warp][g][1] = l[g]; }
        }
    }
    __syncthreads();
    for (int g = warp; g < G; g += ATT_WARPS) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, sm_ml[w][g][0]);
        float ll = 0.0f, acc[EPL];
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[i] = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) {
            const float mw = sm_ml[w][g][0];
            const float c = (mw == -INFINITY) ? 0.0f : expf(mw - mm);
            ll += sm_ml[w][g][1] * c;
#pragma unroll
            for (int i = 0; i < EPL; ++i) acc[i] += sm_o[w][g][lane * EPL + i] * c;
        }
        const int h = kvh * a.group + g0 + g;
        float* dst = a.part + (((int64_t)b * a.H + h) * a.splits + blockIdx.x) * (a.hd + 2);
#pragma unroll
        for (int i = 0; i < EPL; ++i) dst[lane * EPL + i] = acc[i];
        if (lane == 0) { dst[a.hd] = mm; dst[a.hd + 1] = ll; }
    }
}

// grid (H, batch), hd * G threads: merge the splits.  Thread (c, g) adds the splits
// s = g, g + G, ... of output channel c (so up to G * hd loads are in flight instead of
// one dependent chain over all splits), the G partial sums are then added in g order.
// An empty range gives zeros (the reference's sum > 0 guard).
constexpr int MERGE_MAX_THREADS = 1024;
__global__ void __launch_bounds__(MERGE_MAX_THREADS)
attn_decode_merge_kernel(const float* __restrict__ part, float* __restrict__ out, int H, int hd, int splits) {
    __shared__ float s_red[32];
    __shared__ float s_acc[MERGE_MAX_THREADS];
    __shared__ float s_l[MERGE_MAX_THREADS];
    const int h = blockIdx.x, b = blockIdx.y;
    const int G = blockDim.x / hd, c = threadIdx.x % hd, g = threadIdx.x / hd;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float* p = part + ((int64_t)b * H + h) * splits * (hd + 2);
    float mm = -INFINITY;
    for (int s = threadIdx.x; s < splits; s += blockDim.x) mm = fmaxf(mm, p[(int64_t)s * (hd + 2) + hd]);
    mm = warp_max(mm);
    if (lane == 0) s_red[wid] = mm;
    __syncthreads();
    mm = lane < nw ? s_red[lane] : -INFINITY;
    mm = warp_max(mm);
    float ll = 0.0f, acc = 0.0f;
    for (int s = g; s < splits; s += G) {
        const float* ps = p + (int64_t)s * (hd + 2);
        const float w = (ps[hd] == -INFINITY) ? 0.0f : expf(ps[hd] - mm);
        ll += ps[hd + 1] * w;
        acc += ps[c] * w;
    }
    s_acc[threadIdx.x] = acc;
    s_l[threadIdx.x] = ll;
    __syncthreads();
    if (g == 0) {
        for (int k = 1; k < G; ++k) {
            acc += s_acc[k * hd + c];
            ll += s_l[k * hd + c];
        }
        out[((int64_t)b * H + h) * hd + c] = ll > 0.0f ? acc / ll : 0.0f;
    }
}

template <bool HALF, bool PAGED>
// fixed_part / fixed_floats (optional): the split-KV partials go to this caller-supplied
// array instead of the growing workspace, and the number of splits is capped to what it
// holds (every (head, split) record the merge kernel reads is written by the split kernel
// first, so the array needs no clearing between calls).
static int launch_decode(DecodeArgs& a, int batch, int max_len, float* out, float* fixed_part = nullptr,
                         int64_t fixed_floats = 0) {
    const int epl = a.hd / 32;
    const int gblocks = ceil_div(a.group, ATT_GMAX);
    // enough blocks to fill the machine, at least 32 positions per block
    int want = std::max(1, (4 * num_sms()) / std::max(1, a.KV * gblocks * batch));
    if (fixed_part) want = std::min<int64_t>(want, fixed_floats / ((int64_t)batch * a.H * (a.hd + 2)));
    a.splits = std::max(1, std::min(want, ceil_div(std::max(max_len, 1), 32)));
    a.chunk = std::max(1, ceil_div(std::max(max_len, 1), a.splits));
    a.splits = std::max(1, ceil_div(std::max(max_len, 1), a.chunk));
    if (fixed_part) {
        a.part = fixed_part;
    } else {
        void* wsp;
        int rc = workspace(WS_ATTN).ensure((size_t)batch * a.H * a.splits * (a.hd + 2) * sizeof(float) + 256, &wsp);
        if (rc) return rc;
        a.part = static_cast<float*>(wsp);
    }
    const dim3 grid(a.splits, a.KV * gblocks, batch);
    switch (epl) {
        case 1: attn_decode_split_kernel<1, HALF, PAGED><<<grid, ATT_WARPS * 32, 0, stream()>>>(a); break;
        case 2: attn_decode_split_kernel<2, HALF, PAGED><<<grid, ATT_WARPS * 32, 0, stream()>>>(a); break;
        case 4: attn_decode_split_kernel<4, HALF, PAGED><<<grid, ATT_WARPS * 32, 0, stream()>>>(a); break;
        default: attn_decode_split_kernel<8, HALF, PAGED><<<grid, ATT_WARPS * 32, 0, stream()>>>(a); break;
    }
    B200_LAUNCH_CHECK("attn_decode_split_kernel");
    const int merge_groups = std::max(1, std::min(std::min(MERGE_MAX_THREADS / a.hd, 16), a.splits));
    attn_decode_merge_kernel<<<dim3(a.H, batch), a.hd * merge_groups, 0, stream()>>>(a.part, out, a.H, a.hd, a.splits);
    B200_LAUNCH_CHECK("attn_decode_merge_kernel");
    return B200_OK;
}

static int check_hd(const char* who, int hd) {
    B200_REQUIRE(hd == 32 || hd == 64 || hd == 128 || hd == 256, "%s: head_dim must be 32, 64, 128 or 256", who);
    return B200_OK;
}

static int decode_ring(const char* who, const float* q, const void* kc, const void* vc, bool half, float* out,
                       int H, int KV, int hd, int ring_start, int pinned, int cur_len, int cache_max,
                       float scale, int window, float* fixed_part = nullptr, int64_t fixed_floats = 0) {
    // the reference's argument checks (core/attn_cpu.cpp:162-174)
    B200_REQUIRE(H > 0 && KV > 0 && hd > 0, "%s: empty shape", who);
    B200_REQUIRE(H % KV == 0, "%s: H must be a multiple of KV", who);
    B200_REQUIRE(cur_len >= 0 && cache_max >= 0 && cur_len <= cache_max, "%s: length exceeds cache capacity", who);
    B200_REQUIRE(pinned >= 0 && pinned <= cur_len, "%s: pinned prefix out of range", who);
    const int ring_cap = cache_max - pinned;
    if (cur_len > pinned) {
        B200_REQUIRE(ring_cap > 0, "%s: ring has no rolling slots", who);
        B200_REQUIRE(ring_start >= 0 && ring_start < ring_cap, "%s: ring start out of range", who);
    }
    B200_REQUIRE(q && kc && vc && out, "%s: null pointer", who);
    int rc = check_hd(who, hd);
    if (rc) return rc;
    DecodeArgs a{};
    a.q = q; a.kc = kc; a.vc = vc;
    a.H = H; a.KV = KV; a.hd = hd; a.group = H / KV;
    a.cur_len = cur_len;
    a.j0 = (window > 0 && cur_len > window) ? cur_len - window : 0;
    a.ring_start = ring_start; a.pinned = pinned; a.ring_cap = ring_cap > 0 ? ring_cap : 1;
    a.scale = scale;
    const int span = cur_len - a.j0;
    return half ? launch_decode<true, false>(a, 1, span, out, fixed_part, fixed_floats)
                : launch_decode<false, false>(a, 1, span, out, fixed_part, fixed_floats);
}

// ---------------------------------------------------------------------------
// Prefill: one block per (t, h, b); warps stride the keys j0..t with a running
// (max, sum); optional probs output needs the final (max, sum), so it is written
// in a second sweep.
// ---------------------------------------------------------------------------
template <int EPL>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_prefill_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                    float* __restrict__ out, float* __restrict__ probs, int T, int H, int KV, int hd,
                    float scale, int window, const int32_t* __restrict__ seg) {
    __shared__ float sm_o[ATT_WARPS][EPL * 32];
    __shared__ float sm_ml[ATT_WARPS][2];
    __shared__ float s_final[2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (H / KV);
    const int j0 = window > 0 ? max(0, t - window + 1) : 0;
    const int32_t seg_t = seg ? seg[(int64_t)b * T + t] : 0;
    float qv[EPL], o[EPL];
    load_row<EPL, false>(q, (((int64_t)b * T + t) * H + h) * hd, lane, qv);
#pragma unroll
    for (int i = 0; i < EPL; ++i) o[i] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    for (int j = j0 + warp; j <= t; j += ATT_WARPS) {
        if (seg && seg_t >= 0 && seg[(int64_t)b * T + j] != seg_t) continue;
        const int64_t off = (((int64_t)b * T + j) * KV + kvh) * hd;
        float kv[EPL], vv[EPL];
        load_row<EPL, false>(k, off, lane, kv);
        load_row<EPL, false>(v, off, lane, vv);
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) s += qv[i] * kv[i];
        s = warp_sum(s) * scale;
        const float mn = fmaxf(m, s);
        const float corr = expf(m - mn), p = expf(s - mn);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < EPL; ++i) o[i] = o[i] * corr + p * vv[i];
        m = mn;
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) sm_o[warp][lane * EPL + i] = o[i];
    if (lane == 0) { sm_ml[warp][0] = m; sm_ml[warp][1] = l; }
    __syncthreads();
    if (warp == 0) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, sm_ml[w][0]);
        float ll = 0.0f, acc[EPL];
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[i] = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) {
            const float c = (sm_ml[w][0] == -INFINITY) ? 0.0f : expf(sm_ml[w][0] - mm);
            ll += sm_ml[w][1] * c;
#pragma unroll
            for (int i = 0; i < EPL; ++i) acc[i] += sm_o[w][lane * EPL + i] * c;
        }
        const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
        float* dst = out + (((int64_t)b * T + t) * H + h) * hd;
#pragma unroll
        for (int i = 0; i < EPL; ++i) dst[lane * EPL + i] = acc[i] * inv;
        if (lane == 0) { s_final[0] = mm; s_final[1] = inv; }
    }
    if (!probs) return;
    __syncthreads();
    const float mm = s_final[0], inv = s_final[1];
    float* pr = probs + (((int64_t)b * H + h) * T + t) * T;
    for (int j = threadIdx.x; j < T; j += blockDim.x)
        if (j < j0 || j > t) pr[j] = 0.0f;
    for (int j = j0 + warp; j <= t; j += ATT_WARPS) {
        float p = 0.0f;
        if (!(seg && seg_t >= 0 && seg[(int64_t)b * T + j] != seg_t)) {
            float kv[EPL];
            load_row<EPL, false>(k, (((int64_t)b * T + j) * KV + kvh) * hd, lane, kv);
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < EPL; ++i) s += qv[i] * kv[i];
            s = warp_sum(s) * scale;
            p = expf(s - mm) * inv;
        }
        if (lane == 0) pr[j] = p;
    }
}

}  // namespace b200

// attention_flash.cu
namespace b200 {
int attention_flash(const float* q, const float* k, const float* v, float* out, int B, int T, int H, int KV, int hd,
                    float scale, int window, const int32_t* seg);
constexpr int FLASH_MIN_T = 128;
}  // namespace b200

using namespace b200;

extern "C" {

int b200_attention_decode_ring(const float* q, const float* kcache, const float* vcache, float* out,
                               int H, int KV, int hd, int ring_start, int pinned_prefix, int cur_len,
                               int cache_max, float scale, float* scratch, int window) {
    (void)scratch;
    return decode_ring("attention_decode_ring", q, kcache, vcache, false, out, H, KV, hd, ring_start,
                       pinned_prefix, cur_len, cache_max, scale, window);
}
int b200_attention_decode_ring_fp16(const float* q, const uint16_t* kc, const uint16_t* vc, float* out,
                                    int H, int KV, int hd, int ring_start, int pinned_prefix, int cur_len,
                                    int cache_max, float scale, float* scratch, int window) {
    (void)scratch;
    return decode_ring("attention_decode_ring_fp16", q, kc, vc, true, out, H, KV, hd, ring_start,
                       pinned_prefix, cur_len, cache_max, scale, window);
}
int b200_attention_decode_paged_fp16(const float* q, const uint16_t* k_pages, const uint16_t* v_pages,
                                     const int32_t* page_table, const int32_t* seq_lens, float* out,
                                     int batch, int max_pages, int page, int H, int KV, int hd, float scale) {
    if (batch <= 0) return B200_OK;
    B200_REQUIRE(H > 0 && KV > 0 && H % KV == 0, "attention_decode_paged_fp16: H must be a positive multiple of KV");
    B200_REQUIRE(page > 0 && max_pages > 0, "attention_decode_paged_fp16: bad page geometry");
    B200_REQUIRE(q && k_pages && v_pages && page_table && seq_lens && out, "attention_decode_paged_fp16: null pointer");
    int rc = check_hd("attention_decode_paged_fp16", hd);
    if (rc) return rc;
    DecodeArgs a{};
    a.q = q; a.kc = k_pages; a.vc = v_pages;
    a.page_table = page_table; a.seq_lens = seq_lens;
    a.H = H; a.KV = KV; a.hd = hd; a.group = H / KV;
    a.max_pages = max_pages; a.page = page; a.ring_cap = 1;
    a.scale = scale;
    // sequence lengths live on the device: size the splits for the longest possible one
    return launch_decode<true, true>(a, batch, max_pages * page, out);
}

int b200_attention_forward_ex(const float* q, const float* k, const float* v, float* out, float* probs,
                              int B, int T, int H, int KV, int hd, float scale, int window,
                              const int32_t* segment_ids) {
    if (B <= 0 || T <= 0) return B200_OK;
    B200_REQUIRE(H > 0 && KV > 0 && H % KV == 0, "attention_forward_ex: H must be a positive multiple of KV");
    B200_REQUIRE(q && k && v && out, "attention_forward_ex: null pointer");
    B200_REQUIRE(H <= 65535 && B <= 65535, "attention_forward_ex: H and B must be <= 65535");
    int rc = check_hd("attention_forward_ex", hd);
    if (rc) return rc;
    // long sequences without the probability output: the tensor-core kernel (attention_flash.cu)
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (!probs && T >= FLASH_MIN_T && (hd == 64 || hd == 128) && aligned16(q) && aligned16(k) && aligned16(v) &&
        aligned16(out))
        return attention_flash(q, k, v, out, B, T, H, KV, hd, scale, window, segment_ids);
    const dim3 grid(T, H, B);
    switch (hd / 32) {
        case 1: attn_prefill_kernel<1><<<grid, ATT_WARPS * 32, 0, stream()>>>(q, k, v, out, probs, T, H, KV, hd, scale, window, segment_ids); break;
        case 2: attn_prefill_kernel<2><<<grid, ATT_WARPS * 32, 0, stream()>>>(q, k, v, out, probs, T, H, KV, hd, scale, window, segment_ids); break;
        case 4: attn_prefill_kernel<4><<<grid, ATT_WARPS * 32, 0, stream()>>>(q, k, v, out, probs, T, H, KV, hd, scale, window, segment_ids); break;
        default: attn_prefill_kernel<8><<<grid, ATT_WARPS * 32, 0, stream()>>>(q, k, v, out, probs, T, H, KV, hd, scale, window, segment_ids); break;
    }
    B200_LAUNCH_CHECK("attn_prefill_kernel");
    return B200_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// Some hosts of this library cannot tolerate a cudaMalloc on the decode path: a
// serving loop that has handed the whole device to its own pool allocator, a
// latency-critical thread where the implicit device synchronisation of cudaMalloc /
// cudaFree is unacceptable, or code running while another thread captures a stream.
// The regular entry points keep their split-KV partial results in a workspace that
// grows with cudaMalloc on demand; this variant keeps them in a fixed array that is
// part of the library image instead, so it never allocates and never frees.
//
// The array lives in device memory of every GPU that loads the library, from load
// to exit (NOALLOC_FLOATS * 4 bytes = 1 MiB).  Its name is only a host-side handle;
// the device address is looked up once per device with cudaGetSymbolAddress and that
// pointer is what the kernels receive.
// ---------------------------------------------------------------------------
// The cached address does not survive a device reset (cudaDeviceReset) or a re-created
// context: a process that resets a device must not call this entry point afterwards.
namespace b200 {
constexpr int NOALLOC_FLOATS = 256 * 1024;
constexpr int NOALLOC_MAX_DEVICES = 64;
static __device__ __align__(256) float g_noalloc_partials[NOALLOC_FLOATS];
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES];   // device address of the array, per device
static std::once_flag g_noalloc_once[NOALLOC_MAX_DEVICES];
}  // namespace b200

extern "C" int b200_attention_decode_ring_fp16_noalloc(const float* q, const uint16_t* kc, const uint16_t* vc,
                                                       float* out, int H, int KV, int hd, int ring_start,
                                                       int pinned_prefix, int cur_len, int cache_max,
                                                       float scale, int window) {
    const char* who = "attention_decode_ring_fp16_noalloc";
    // The fixed scratch bounds the problem: at least one split of (hd + 2) floats per head.
    B200_REQUIRE(H > 0 && hd > 0 && (int64_t)H * (hd + 2) <= NOALLOC_FLOATS,
                 "%s: H * (head_dim + 2) = %lld floats exceeds the built-in scratch of %d floats; use "
                 "attention_decode_ring_fp16 for this shape", who, (long long)H * (hd + 2), NOALLOC_FLOATS);
    // One-time set-up per device, with that device current: resolve the array's device
    // address (first callers of a device race to here; exactly one of them looks it up).
    // This first call should happen outside any stream capture.
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < NOALLOC_MAX_DEVICES, "%s: device index %d not supported", who, dev);
    cudaError_t lookup = cudaSuccess;
    std::call_once(g_noalloc_once[dev], [&] {
        float* p = nullptr;
        lookup = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_partials);
        g_noalloc_ptr[dev] = lookup == cudaSuccess ? p : nullptr;
    });
    if (lookup != cudaSuccess) return cuda_status(lookup, "attention_decode_ring_fp16_noalloc: cudaGetSymbolAddress");
    B200_REQUIRE(g_noalloc_ptr[dev], "%s: the built-in scratch could not be located on device %d", who, dev);
    // argument checks, split sizing and dispatch are the allocating entry point's
    return decode_ring(who, q, kc, vc, true, out, H, KV, hd, ring_start, pinned_prefix, cur_len, cache_max, scale, window,
                       g_noalloc_ptr[dev], NOALLOC_FLOATS);
}
