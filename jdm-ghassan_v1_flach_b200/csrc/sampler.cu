// The sampling tail on the device: what the reference does on the host after every
// token (inference/sampler.cpp: penalties, n-gram ban, greedy / top-k / top-p / min-p
// draw from the generator of core/rng.h) and the cross-entropy behind perplexity scoring
// (Generator::score_tokens, inference/generator.cpp:1217-1294; core/math_cpu.cpp:560-612).
// The generator state, the token history and the pick stay in device memory, so a
// sampled decode loop needs no host round trip and can be replayed as a CUDA graph.
//
// Arithmetic follows the host code step by step: probabilities are exp() of the fp32
// value (v - max) * (1 / temperature) evaluated in double, sums run in double in candidate
// order on one thread (the candidate sets are small), and the draw consumes one 24-bit
// uniform of the xoshiro256** stream exactly where the host does.  Candidates of equal
// value are ordered by ascending id (the host's std::sort leaves that order open).
#include <algorithm>
#include <cmath>
#include <cstring>

#include "sampler.cuh"

namespace b200 {

constexpr int HIST_MAX = 8192;          // Generator::HIST_MAX, inference/generator.h:96
constexpr int CAND_SMEM_MAX = 2048;     // candidate sets up to this size are sorted and drawn in shared memory

// ---- core/rng.h:8-41 --------------------------------------------------------
__host__ __device__ inline uint64_t rotl64(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
__host__ __device__ inline void rng_seed_state(uint64_t seed, uint64_t* s) {
    for (int i = 0; i < 4; ++i) {
        seed += 0x9E3779B97F4A7C15ULL;
        uint64_t z = seed;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
        s[i] = z ^ (z >> 31);
    }
}
__device__ inline uint64_t rng_next(uint64_t* s) {
    const uint64_t r = rotl64(s[1] * 5, 7) * 9;
    const uint64_t t = s[1] << 17;
    s[2] ^= s[0];
    s[3] ^= s[1];
    s[1] ^= s[2];
    s[0] ^= s[3];
    s[2] ^= t;
    s[3] = rotl64(s[3], 45);
    return r;
}
__device__ inline float rng_uniform(uint64_t* s) { return (float)((double)(rng_next(s) >> 40) * (1.0 / 16777216.0)); }

// ---- candidates as sortable words -------------------------------------------
// High word: the value mapped so that unsigned order is numeric order (-0 as +0); low
// word: ~id, so that a descending sort puts equal values in ascending id order.
__device__ __forceinline__ uint64_t cand_key(float v, int id) {
    if (v == 0.0f) v = 0.0f;
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((uint64_t)u << 32) | (uint32_t)(~(uint32_t)id);
}
__device__ __forceinline__ float key_value(uint64_t k) {
    uint32_t u = (uint32_t)(k >> 32);
    u = (u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u;
    return __uint_as_float(u);
}
__device__ __forceinline__ int key_id(uint64_t k) { return (int)(~(uint32_t)k); }

// Block-wide bitonic sort, descending; n2 a power of two; keys in shared or global memory.
__device__ void bitonic_desc(uint64_t* keys, int n2) {
    for (int k = 2; k <= n2; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < n2; i += blockDim.x) {
                const int p = i ^ j;
                if (p > i) {
                    const uint64_t a = keys[i], b = keys[p];
                    const bool desc = (i & k) == 0;
                    if (desc ? a < b : a > b) {
                        keys[i] = b;
                        keys[p] = a;
                    }
                }
            }
            __syncthreads();
        }
    }
}

// Sampler::draw_from_scratch (inference/sampler.cpp:206-266) over n candidates sorted in
// descending order; probs: n doubles of scratch.  Every thread of the block calls it; the
// pick is returned to thread 0 only.
__device__ int draw_sorted(const uint64_t* keys, double* probs, int n, float temperature, float top_p, float min_p,
                           uint64_t* rng) {
    if (!(temperature > 0.0f)) return key_id(keys[0]);
    const float inv_t = __fdiv_rn(1.0f, temperature);
    const float mx = key_value(keys[0]);
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        probs[i] = exp((double)__fmul_rn(__fsub_rn(key_value(keys[i]), mx), inv_t));
    __syncthreads();
    __shared__ double s_sum;
    if (threadIdx.x == 0) {
        double sum = 0.0;
        for (int i = 0; i < n; ++i) sum += probs[i];
        s_sum = sum;
    }
    __syncthreads();
    const double sum = s_sum;
    if (!isfinite(sum) || sum <= 0.0) return key_id(keys[0]);
    for (int i = threadIdx.x; i < n; i += blockDim.x) probs[i] = probs[i] / sum;
    __syncthreads();
    if (threadIdx.x != 0) return -1;
    int limit = n;
    if (min_p > 0.0f) {
        const double thresh = (double)min_p * probs[0];
        int m = 0;
        while (m < n && probs[m] >= thresh) ++m;
        limit = m > 1 ? m : 1;
    }
    if (top_p > 0.0f && top_p < 1.0f) {
        double cum = 0.0;
        int m = 0;
        while (m < limit) {
            cum += probs[m];
            ++m;
            if (cum >= (double)top_p) break;
        }
        limit = m > 1 ? m : 1;
    }
    double renorm = 0.0;
    for (int i = 0; i < limit; ++i) renorm += probs[i];
    const double r = (double)rng_uniform(rng) * renorm;
    double acc = 0.0;
    for (int i = 0; i < limit; ++i) {
        acc += probs[i];
        if (r <= acc) return key_id(keys[i]);
    }
    return key_id(keys[limit - 1]);
}

// Candidate sets of up to CAND_SMEM_MAX entries: sort and draw in shared memory.  Input
// either as (vals, ids) [rows, K] or as keys [rows, K].
__global__ void __launch_bounds__(256) draw_small_kernel(const float* __restrict__ vals, const int32_t* __restrict__ ids,
                                                         const uint64_t* __restrict__ keys_in, int K, float temperature,
                                                         float top_p, float min_p, uint64_t* __restrict__ rng,
                                                         int32_t* __restrict__ next) {
    __shared__ uint64_t keys[CAND_SMEM_MAX];
    __shared__ double probs[CAND_SMEM_MAX];
    const int r = blockIdx.x;
    int n2 = 1;
    while (n2 < K) n2 <<= 1;
    for (int i = threadIdx.x; i < n2; i += blockDim.x) {
        uint64_t k = 0;      // below every real candidate
        if (i < K) k = keys_in ? keys_in[(int64_t)r * K + i] : cand_key(vals[(int64_t)r * K + i], ids[(int64_t)r * K + i]);
        keys[i] = k;
    }
    __syncthreads();
    bitonic_desc(keys, n2);
    const int pick = draw_sorted(keys, probs, K, temperature, top_p, min_p, rng + 4 * r);
    if (threadIdx.x == 0) next[r] = pick;
}

// The K largest of a row by K passes (ties to the lower id), as sortable words.
__global__ void __launch_bounds__(1024) topk_rounds_kernel(const float* __restrict__ logits, int V, int K,
                                                           uint64_t* __restrict__ keys) {
    __shared__ uint64_t sm[32];
    __shared__ uint64_t prev;
    const float* row = logits + (int64_t)blockIdx.x * V;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (threadIdx.x == 0) prev = ~0ull;
    __syncthreads();
    for (int r = 0; r < K; ++r) {
        const uint64_t p = prev;
        uint64_t mine = 0;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const uint64_t c = cand_key(row[i], i);
            if (c < p && c > mine) mine = c;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const uint64_t other = __shfl_xor_sync(0xffffffffu, mine, o);
            mine = other > mine ? other : mine;
        }
        if (lane == 0) sm[wid] = mine;
        __syncthreads();
        if (wid == 0) {
            uint64_t t = sm[lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const uint64_t other = __shfl_xor_sync(0xffffffffu, t, o);
                t = other > t ? other : t;
            }
            if (lane == 0) {
                keys[(int64_t)blockIdx.x * K + r] = t;
                prev = t;
            }
        }
        __syncthreads();
    }
}

// Whole rows sorted in global scratch (keys [rows, n2]) and drawn from the first K.
__global__ void __launch_bounds__(1024) sort_draw_kernel(const float* __restrict__ logits, int V, int n2, int K,
                                                         uint64_t* __restrict__ keys_ws, double* __restrict__ probs_ws,
                                                         float temperature, float top_p, float min_p,
                                                         uint64_t* __restrict__ rng, int32_t* __restrict__ next) {
    const int r = blockIdx.x;
    uint64_t* keys = keys_ws + (int64_t)r * n2;
    double* probs = probs_ws + (int64_t)r * n2;
    const float* row = logits + (int64_t)r * V;
    for (int i = threadIdx.x; i < n2; i += blockDim.x) keys[i] = i < V ? cand_key(row[i], i) : 0ull;
    __syncthreads();
    bitonic_desc(keys, n2);
    const int pick = draw_sorted(keys, probs, K, temperature, top_p, min_p, rng + 4 * r);
    if (threadIdx.x == 0) next[r] = pick;
}

// Sampler::sample without any filter (inference/sampler.cpp:143-167): the first largest
// logit changes places with element 0 and one pass over the vocabulary draws.  The
// running sum is formed per contiguous slice of that order and the slices are then added
// in order (the host adds element by element; the results differ in the last bits only).
__global__ void __launch_bounds__(1024) softmax_draw_kernel(const float* __restrict__ logits, int V, float temperature,
                                                            uint64_t* __restrict__ rng, int32_t* __restrict__ next) {
    __shared__ uint64_t sm[32];
    __shared__ double part[1024];
    __shared__ int s_bi;
    const int r = blockIdx.x;
    const float* row = logits + (int64_t)r * V;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint64_t mine = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const uint64_t c = cand_key(row[i], i);
        mine = c > mine ? c : mine;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const uint64_t other = __shfl_xor_sync(0xffffffffu, mine, o);
        mine = other > mine ? other : mine;
    }
    if (lane == 0) sm[wid] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint64_t t = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t = sm[w] > t ? sm[w] : t;
        s_bi = key_id(t);
    }
    __syncthreads();
    const int bi = s_bi;
    const float mx = row[bi];
    const float inv_t = __fdiv_rn(1.0f, temperature);
    const int L = (V + (int)blockDim.x - 1) / (int)blockDim.x;
    auto elem = [&](int pos) { return pos == 0 ? bi : (pos == bi ? 0 : pos); };
    auto prob = [&](int pos) { return exp((double)__fmul_rn(__fsub_rn(row[elem(pos)], mx), inv_t)); };
    {
        double s = 0.0;
        const int lo = threadIdx.x * L, hi = min(V, lo + L);
        for (int pos = lo; pos < hi; ++pos) s += prob(pos);
        part[threadIdx.x] = s;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    double sum = 0.0;
    for (int c = 0; c < (int)blockDim.x; ++c) sum += part[c];
    if (!isfinite(sum) || sum <= 0.0) {
        next[r] = bi;
        return;
    }
    const double rr = (double)rng_uniform(rng + 4 * r) * sum;
    double acc = 0.0;
    int pick = elem(V - 1);
    for (int c = 0; c < (int)blockDim.x; ++c) {
        if (rr <= acc + part[c] || c == (int)blockDim.x - 1) {
            const int lo = c * L, hi = min(V, lo + L);
            bool found = false;
            for (int pos = lo; pos < hi; ++pos) {
                acc += prob(pos);
                if (rr <= acc) {
                    pick = elem(pos);
                    found = true;
                    break;
                }
            }
            if (found) break;
            // rounding put the crossing just behind this slice: carry on with the next one
            continue;
        }
        acc += part[c];
    }
    next[r] = pick;
}

// Greedy branch of Sampler::sample (inference/sampler.cpp:131-141): the largest finite
// logit, the first of equals; when nothing is finite, the largest by '>' from element 0.
__global__ void __launch_bounds__(1024) greedy_rows_kernel(const float* __restrict__ logits, int V,
                                                           int32_t* __restrict__ next) {
    __shared__ uint64_t sm[32];
    const float* row = logits + (int64_t)blockIdx.x * V;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint64_t mine = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (isfinite(v)) {
            const uint64_t c = cand_key(v, i);
            mine = c > mine ? c : mine;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const uint64_t other = __shfl_xor_sync(0xffffffffu, mine, o);
        mine = other > mine ? other : mine;
    }
    if (lane == 0) sm[wid] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint64_t t = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t = sm[w] > t ? sm[w] : t;
        int best;
        if (t != 0) {
            best = key_id(t);
        } else {
            best = 0;
            for (int i = 1; i < V; ++i)
                if (row[i] > row[best]) best = i;
        }
        next[blockIdx.x] = best;
    }
}

// Penalties over the window and the n-gram ban over the whole history
// (Sampler::apply_penalties :75-107, ban_no_repeat_ngram :109-124).  One block per row;
// dynamic shared memory: the row's available history.
__global__ void __launch_bounds__(1024) penalty_kernel(float* __restrict__ logits, int V, const int32_t* __restrict__ hist,
                                                       int cap, const int32_t* __restrict__ totals, int window_cfg,
                                                       float rep, float freq, float pres, int ngram) {
    extern __shared__ int32_t h[];
    const int r = blockIdx.x;
    float* row = logits + (int64_t)r * V;
    const int total = totals[r];
    const int avail = min(min(total, cap), HIST_MAX);
    const int32_t* ring = hist + (int64_t)r * cap;
    for (int j = threadIdx.x; j < avail; j += blockDim.x) h[j] = ring[(total - avail + j) % cap];
    __syncthreads();
    if (avail == 0) return;
    const bool use_rep = rep != 1.0f, use_freq = freq != 0.0f, use_pres = pres != 0.0f;
    if (use_rep || use_freq || use_pres) {
        const int window = window_cfg > 0 ? min(avail, window_cfg) : avail;
        const int w0 = avail - window;
        for (int i = w0 + threadIdx.x; i < avail; i += blockDim.x) {
            const int32_t tok = h[i];
            if (tok < 0 || tok >= V) continue;
            int count = 0;
            bool first = true;
            for (int j = w0; j < avail; ++j) {
                if (h[j] == tok) {
                    if (j < i) { first = false; break; }
                    ++count;
                }
            }
            if (!first) continue;
            float l = row[tok];
            if (use_rep) l = (l > 0.0f) ? __fdiv_rn(l, rep) : __fmul_rn(l, rep);
            if (use_freq) l = __fsub_rn(l, __fmul_rn(freq, (float)count));
            if (use_pres) l = __fsub_rn(l, pres);
            row[tok] = l;
        }
    }
    __syncthreads();
    if (ngram > 0 && avail >= ngram - 1) {
        const int pre = ngram - 1;
        for (int i = threadIdx.x; i + ngram <= avail; i += blockDim.x) {
            bool match = true;
            for (int k = 0; k < pre; ++k)
                if (h[i + k] != h[avail - pre + k]) { match = false; break; }
            if (!match) continue;
            const int32_t nxt = h[i + pre];
            if (nxt >= 0 && nxt < V) row[nxt] = -1e30f;
        }
    }
}

// seq_off (optional): row r's tokens are tokens[seq_off[r] .. seq_off[r + 1]) instead of
// tokens[r T .. (r + 1) T).
__global__ void history_push_kernel(int32_t* __restrict__ hist, int cap, int32_t* __restrict__ totals,
                                    const int32_t* __restrict__ tokens, int rows, int T,
                                    const int32_t* __restrict__ seq_off) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    if (seq_off) {
        tokens += seq_off[r] - (int64_t)r * (seq_off[r + 1] - seq_off[r]);
        T = seq_off[r + 1] - seq_off[r];
    }
    int total = totals[r];
    const int first = T > cap ? T - cap : 0;       // older prompt tokens would be overwritten anyway
    total += first;
    for (int t = first; t < T; ++t) {
        hist[(int64_t)r * cap + total % cap] = tokens[(int64_t)r * T + t];
        ++total;
    }
    totals[r] = total;
}

__global__ void rng_seed_kernel(uint64_t seed, uint64_t* __restrict__ state, int streams) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < streams) rng_seed_state(seed + (uint64_t)i, state + 4 * i);
}
__global__ void rng_uniform_kernel(uint64_t* __restrict__ state, float* __restrict__ out, int n) {
    if (blockIdx.x == 0 && threadIdx.x == 0)
        for (int i = 0; i < n; ++i) out[i] = rng_uniform(state);
}

// ---- cross-entropy ------------------------------------------------------------
__global__ void __launch_bounds__(512) ce_rows_kernel(const float* __restrict__ logits, const int32_t* __restrict__ targets,
                                                      int V, float z_scale, double* __restrict__ losses,
                                                      double* __restrict__ acc) {
    __shared__ double red[32];
    __shared__ float redf[32];
    const int64_t r = blockIdx.x;
    const int32_t tgt = targets[r];
    if (tgt < 0 || tgt >= V) {
        if (threadIdx.x == 0) {
            losses[r] = 0.0;
            if (tgt >= V) reinterpret_cast<unsigned long long*>(acc)[2] = 1ull;
        }
        return;
    }
    const float* row = logits + r * V;
    float mx = -INFINITY;
    for (int j = threadIdx.x; j < V; j += blockDim.x) mx = fmaxf(mx, row[j]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) redf[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = redf[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, redf[w]);
    double s = 0.0;
    for (int j = threadIdx.x; j < V; j += blockDim.x) s += exp((double)__fsub_rn(row[j], mx));
    s = block_sum_d(s, red);
    if (threadIdx.x == 0) {
        const double logZ = log(s) + (double)mx;
        double l = logZ - (double)row[tgt];
        if (z_scale != 0.0f) l += (double)z_scale * logZ * logZ;
        losses[r] = l;
    }
}
// Fixed-order sum of the row losses (so that the result does not depend on scheduling).
__global__ void __launch_bounds__(1024) ce_fold_kernel(const double* __restrict__ losses, const int32_t* __restrict__ targets,
                                                       int64_t n, int V, double* __restrict__ acc) {
    __shared__ double red[32];
    __shared__ double redc[32];
    double s = 0.0, c = 0.0;
    const int64_t L = (n + blockDim.x - 1) / blockDim.x;
    const int64_t lo = threadIdx.x * L, hi = lo + L < n ? lo + L : n;
    for (int64_t i = lo; i < hi; ++i) {
        s += losses[i];
        c += (targets[i] >= 0 && targets[i] < V) ? 1.0 : 0.0;
    }
    s = block_sum_d(s, red);
    c = block_sum_d(c, redc);
    if (threadIdx.x == 0) {
        acc[0] += s;
        reinterpret_cast<long long*>(acc)[1] += (long long)c;
    }
}

// ---- host side ------------------------------------------------------------------
bool sampling_is_greedy(const b200_sampling& c) { return c.greedy != 0 || c.temperature <= 0.0f || c.top_k == 1; }

static bool no_filter(const b200_sampling& c, int V) {
    return (c.top_k <= 0 || c.top_k >= V) && (c.top_p <= 0.0f || c.top_p >= 1.0f) && c.min_p <= 0.0f;
}
static int pow2_at_least(int v) {
    int n = 1;
    while (n < v) n <<= 1;
    return n;
}

size_t sample_workspace_bytes(const b200_sampling& c, int V, int rows) {
    if (sampling_is_greedy(c) || no_filter(c, V)) return 256;
    const int k = (c.top_k > 0 && c.top_k < V) ? c.top_k : V;
    if (k <= SAMPLE_TOPK_ROUNDS_MAX) return (size_t)rows * k * 8 + 256;
    return (size_t)rows * pow2_at_least(V) * 16 + 256;
}

int sample_rows(float* logits, int V, int rows, const int32_t* hist, int cap, const int32_t* totals, const b200_sampling& c,
                uint64_t* rng, int32_t* next, void* ws) {
    cudaStream_t st = stream();
    const bool penalties = c.repetition_penalty != 1.0f || c.frequency_penalty != 0.0f || c.presence_penalty != 0.0f;
    if (hist && totals && (penalties || c.no_repeat_ngram > 0)) {
        const size_t smem = (size_t)std::min(cap, HIST_MAX) * 4;
        penalty_kernel<<<rows, 1024, smem, st>>>(logits, V, hist, cap, totals, c.repetition_window, c.repetition_penalty,
                                                 c.frequency_penalty, c.presence_penalty, c.no_repeat_ngram);
        B200_LAUNCH_CHECK("penalty_kernel");
    }
    if (sampling_is_greedy(c)) {
        greedy_rows_kernel<<<rows, 1024, 0, st>>>(logits, V, next);
        B200_LAUNCH_CHECK("greedy_rows_kernel");
        return B200_OK;
    }
    if (no_filter(c, V)) {
        softmax_draw_kernel<<<rows, 1024, 0, st>>>(logits, V, c.temperature, rng, next);
        B200_LAUNCH_CHECK("softmax_draw_kernel");
        return B200_OK;
    }
    const int k = (c.top_k > 0 && c.top_k < V) ? c.top_k : V;
    if (k <= SAMPLE_TOPK_ROUNDS_MAX) {
        uint64_t* keys = static_cast<uint64_t*>(ws);
        topk_rounds_kernel<<<rows, 1024, 0, st>>>(logits, V, k, keys);
        B200_LAUNCH_CHECK("topk_rounds_kernel");
        draw_small_kernel<<<rows, 256, 0, st>>>(nullptr, nullptr, keys, k, c.temperature, c.top_p, c.min_p, rng, next);
        B200_LAUNCH_CHECK("draw_small_kernel");
        return B200_OK;
    }
    const int n2 = pow2_at_least(V);
    uint64_t* keys = static_cast<uint64_t*>(ws);
    double* probs = reinterpret_cast<double*>(keys + (size_t)rows * n2);
    sort_draw_kernel<<<rows, 1024, 0, st>>>(logits, V, n2, k, keys, probs, c.temperature, c.top_p, c.min_p, rng, next);
    B200_LAUNCH_CHECK("sort_draw_kernel");
    return B200_OK;
}

int history_push(int32_t* hist, int cap, int32_t* totals, const int32_t* tokens, int rows) {
    return history_push_prompt(hist, cap, totals, tokens, rows, 1, nullptr);
}
int history_push_prompt(int32_t* hist, int cap, int32_t* totals, const int32_t* tokens, int rows, int T,
                        const int32_t* seq_off) {
    history_push_kernel<<<ceil_div(rows, 128), 128, 0, stream()>>>(hist, cap, totals, tokens, rows, T, seq_off);
    B200_LAUNCH_CHECK("history_push_kernel");
    return B200_OK;
}

int cross_entropy_accumulate(const float* logits, const int32_t* targets, int64_t n, int V, float z_scale, double* losses,
                             double* acc) {
    ce_rows_kernel<<<(unsigned)n, 512, 0, stream()>>>(logits, targets, V, z_scale, losses, acc);
    B200_LAUNCH_CHECK("ce_rows_kernel");
    ce_fold_kernel<<<1, 1024, 0, stream()>>>(losses, targets, n, V, acc);
    B200_LAUNCH_CHECK("ce_fold_kernel");
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

// SamplingConfig::validate, inference/sampler.cpp:36-73.
int b200_sampling_validate(b200_sampling* c) {
    B200_REQUIRE(c, "sampling_validate: null pointer");
    if (!std::isfinite(c->temperature) || c->temperature < 0.0f) c->temperature = 0.0f;
    if (c->temperature > 5.0f) c->temperature = 5.0f;
    if (!std::isfinite(c->top_p) || c->top_p < 0.0f) c->top_p = 1.0f;
    if (c->top_p > 1.0f) c->top_p = 1.0f;
    if (!std::isfinite(c->min_p) || c->min_p < 0.0f) c->min_p = 0.0f;
    if (c->min_p >= 1.0f) c->min_p = 0.0f;
    if (c->top_k < 0) c->top_k = 0;
    if (c->top_k > 2048) c->top_k = 2048;
    if (!std::isfinite(c->repetition_penalty) || c->repetition_penalty <= 0.0f) c->repetition_penalty = 1.0f;
    if (c->repetition_penalty > 5.0f) c->repetition_penalty = 5.0f;
    if (!std::isfinite(c->frequency_penalty)) c->frequency_penalty = 0.0f;
    if (!std::isfinite(c->presence_penalty)) c->presence_penalty = 0.0f;
    c->frequency_penalty = std::min(5.0f, std::max(-5.0f, c->frequency_penalty));
    c->presence_penalty = std::min(5.0f, std::max(-5.0f, c->presence_penalty));
    c->repetition_window = std::min(8192, std::max(0, c->repetition_window));
    if (c->no_repeat_ngram < 0) c->no_repeat_ngram = 0;
    if (c->no_repeat_ngram == 1) c->no_repeat_ngram = 2;
    if (c->no_repeat_ngram > 8) c->no_repeat_ngram = 8;
    return B200_OK;
}

int b200_rng_seed(uint64_t seed, uint64_t* state_dev, int streams) {
    B200_REQUIRE(state_dev && streams >= 1, "rng_seed: bad arguments");
    rng_seed_kernel<<<ceil_div(streams, 128), 128, 0, stream()>>>(seed, state_dev, streams);
    B200_LAUNCH_CHECK("rng_seed_kernel");
    return B200_OK;
}

int b200_rng_uniform(uint64_t* state_dev, float* out_dev, int n) {
    B200_REQUIRE(state_dev && out_dev && n >= 0, "rng_uniform: bad arguments");
    if (n == 0) return B200_OK;
    rng_uniform_kernel<<<1, 32, 0, stream()>>>(state_dev, out_dev, n);
    B200_LAUNCH_CHECK("rng_uniform_kernel");
    return B200_OK;
}

int b200_sample_candidates(const float* vals_dev, const int32_t* ids_dev, int K, int rows, const b200_sampling* cfg,
                           uint64_t* rng_state_dev, int32_t* next_dev) {
    B200_REQUIRE(vals_dev && ids_dev && cfg && rng_state_dev && next_dev, "sample_candidates: null pointer");
    B200_REQUIRE(K >= 1 && K <= CAND_SMEM_MAX && rows >= 1, "sample_candidates: K must be in [1, %d]", CAND_SMEM_MAX);
    draw_small_kernel<<<rows, 256, 0, stream()>>>(vals_dev, ids_dev, nullptr, K, cfg->temperature, cfg->top_p, cfg->min_p,
                                                  rng_state_dev, next_dev);
    B200_LAUNCH_CHECK("draw_small_kernel");
    return B200_OK;
}

int b200_sample_logits(float* logits_dev, int V, int rows, const int32_t* hist_dev, int hist_stride,
                       const int32_t* hist_len_dev, const b200_sampling* cfg, uint64_t* rng_state_dev, int32_t* next_dev) {
    B200_REQUIRE(logits_dev && cfg && rng_state_dev && next_dev, "sample_logits: null pointer");
    B200_REQUIRE(V >= 1 && rows >= 1, "sample_logits: bad sizes");
    B200_REQUIRE((hist_dev == nullptr) == (hist_len_dev == nullptr), "sample_logits: history and its lengths go together");
    B200_REQUIRE(!hist_dev || (hist_stride >= 1 && hist_stride <= HIST_MAX),
                 "sample_logits: at most %d history tokens per row", HIST_MAX);
    b200_sampling c = *cfg;
    b200_sampling_validate(&c);
    void* ws;
    int rc = workspace(WS_SAMPLE).ensure(sample_workspace_bytes(c, V, rows), &ws);
    if (rc) return rc;
    return sample_rows(logits_dev, V, rows, hist_dev, hist_stride, hist_len_dev, c, rng_state_dev, next_dev, ws);
}

int b200_softmax_cross_entropy(const float* logits, const int32_t* targets, float* dlogits, int64_t n, int V,
                               double* out_loss_sum, int64_t* out_count, float z_scale) {
    if (n <= 0) {
        if (out_loss_sum) *out_loss_sum = 0.0;
        if (out_count) *out_count = 0;
        return B200_OK;
    }
    if (dlogits) return fail(B200_EUNSUPPORTED, "softmax_cross_entropy: the gradient is a training op this library does not provide");
    B200_REQUIRE(logits && targets && V >= 1 && n <= 0x7fffffff, "softmax_cross_entropy: bad arguments");
    void* ws;
    int rc = workspace(WS_SAMPLE).ensure((size_t)n * 8 + 256, &ws);
    if (rc) return rc;
    double* acc = static_cast<double*>(ws);
    double* losses = acc + 4;
    B200_CUDA(cudaMemsetAsync(acc, 0, 32, stream()));
    rc = cross_entropy_accumulate(logits, targets, n, V, z_scale, losses, acc);
    if (rc) return rc;
    unsigned long long host[3];
    B200_CUDA(cudaMemcpyAsync(host, acc, 24, cudaMemcpyDeviceToHost, stream()));
    B200_CUDA(cudaStreamSynchronize(stream()));
    B200_REQUIRE(host[2] == 0, "softmax_cross_entropy: a target is outside the vocabulary of %d", V);
    double sum;
    memcpy(&sum, &host[0], 8);
    if (out_loss_sum) *out_loss_sum = sum;
    if (out_count) *out_count = (int64_t)host[1];
    return B200_OK;
}

}  // extern "C"
