// Small memory-bound ops of the forward step: residual/elementwise, embedding
// gather, RMSNorm, cached RoPE, SwiGLU and the sampling tail.
// Reference: core/math_cpu.cpp (the arithmetic that is matched) and
// cuda/kernels.cu:775-1076,1260-1496 (the kernels that are replaced).
#include <algorithm>
#include <cfloat>

#include "common.cuh"

namespace b200 {

static inline int flat_grid(int64_t n, int per_thread = 1) {
    const int64_t blocks = ceil_div64(ceil_div64(n, per_thread), 256);
    return (int)std::max<int64_t>(1, std::min<int64_t>(blocks, (int64_t)num_sms() * 16));
}

#define GRID_STRIDE(i, n)                                                       \
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < (n); \
         i += (int64_t)gridDim.x * blockDim.x)

__global__ void add_kernel(const float* a, const float* b, float* out, int64_t n) {
    GRID_STRIDE(i, n) out[i] = a[i] + b[i];
}
__global__ void add_bias_kernel(const float* __restrict__ b, float* __restrict__ y, int64_t total, int cols) {
    GRID_STRIDE(i, total) y[i] += b[i % cols];
}
__global__ void scale_kernel(float* a, float s, int64_t n) { GRID_STRIDE(i, n) a[i] *= s; }
__global__ void swiglu_kernel(const float* __restrict__ g, const float* __restrict__ u,
                              float* __restrict__ out, int64_t n) {
    GRID_STRIDE(i, n) out[i] = silu_acc(g[i]) * u[i];
}

// Row gather; an id outside [0, vocab) gives a zero row (core/math_cpu.cpp:213-241).
template <bool HALF>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const void* __restrict__ table,
                                 float* __restrict__ out, int dim, int vocab) {
    const int64_t t = blockIdx.x;
    const int32_t id = ids[t];
    float* o = out + t * dim;
    const bool ok = id >= 0 && id < vocab;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = 0.0f;
        if (ok) {
            if (HALF) v = half_bits_to_float(static_cast<const uint16_t*>(table)[(int64_t)id * dim + i]);
            else v = static_cast<const float*>(table)[(int64_t)id * dim + i];
        }
        o[i] = v;
    }
}

// One block per row.  Sum of squares in double and inv = 1/sqrt(mean + eps) in
// double rounded to float, as core/math_cpu.cpp:299-316; non-finite inv -> 0.
// x may alias out (each element is read before it is written by the same thread).
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* x, const float* __restrict__ w,
                                                      float* out, float* rrms, int dim, float eps) {
    __shared__ double red[32];
    const int64_t r = blockIdx.x;
    const float* xr = x + r * dim;
    double ss = 0.0;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const double v = (double)xr[i];
        ss += v * v;
    }
    ss = block_sum_d(ss, red);
    const double inv_d = 1.0 / sqrt(ss / (double)dim + (double)eps);
    const float inv = isfinite(inv_d) ? (float)inv_d : 0.0f;
    if (rrms && threadIdx.x == 0) rrms[r] = inv;
    float* o = out + r * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = xr[i] * inv * w[i];
}

// One thread per (token, pair index); angle = float(double(pos) * double(inv_freq))
// as core/math_cpu.cpp:464-496.
__global__ void rope_cached_kernel(float* q, float* k, const int32_t* __restrict__ pos,
                                   const float* __restrict__ inv_freq, int64_t ntok, int n_heads,
                                   int n_kv, int head_dim, int rope_type) {
    const int half = head_dim / 2;
    const int64_t total = ntok * half;
    GRID_STRIDE(idx, total) {
        const int64_t t = idx / half;
        const int i = (int)(idx - t * half);
        const float ang = (float)((double)pos[t] * (double)inv_freq[i]);
        float s, c;
        sincosf(ang, &s, &c);
        const int ia = rope_type == 1 ? i : 2 * i;
        const int ib = rope_type == 1 ? i + half : 2 * i + 1;
        if (q)
            for (int h = 0; h < n_heads; ++h) {
                float* row = q + (t * n_heads + h) * head_dim;
                const float a = row[ia], b = row[ib];
                row[ia] = a * c - b * s;
                row[ib] = a * s + b * c;
            }
        if (k)
            for (int h = 0; h < n_kv; ++h) {
                float* row = k + (t * n_kv + h) * head_dim;
                const float a = row[ia], b = row[ib];
                row[ia] = a * c - b * s;
                row[ib] = a * s + b * c;
            }
    }
}

// ---- sampling tail ---------------------------------------------------------
struct Best {
    float v;
    int i;
};
// a is better than b: larger value, ties to the lower index.
__device__ __forceinline__ bool better(const Best& a, const Best& b) {
    if (a.i < 0) return false;
    if (b.i < 0) return true;
    return a.v > b.v || (a.v == b.v && a.i < b.i);
}
__device__ __forceinline__ Best block_best(Best mine, Best* sm) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, mine.v, o), __shfl_xor_sync(0xffffffffu, mine.i, o)};
        if (better(other, mine)) mine = other;
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) sm[wid] = mine;
    __syncthreads();
    Best t = lane < nw ? sm[lane] : Best{0.0f, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
        if (better(other, t)) t = other;
    }
    return t;
}

// Greedy pick (core/math_cpu.cpp:709-722): largest finite logit, ties to the lowest
// id; if no logit is finite, the largest by '>' starting from id 0.
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int V,
                                                      int32_t* __restrict__ out) {
    __shared__ Best sm[32];
    Best mine{0.0f, -1};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = logits[i];
        if (isfinite(v)) {
            const Best c{v, i};
            if (better(c, mine)) mine = c;
        }
    }
    Best b = block_best(mine, sm);
    if (b.i < 0 && threadIdx.x == 0) {
        // nothing finite (degenerate): the reference's serial scan, NaN compares false
        int best = 0;
        for (int i = 1; i < V; ++i)
            if (logits[i] > logits[best]) best = i;
        b.i = best;
    }
    if (threadIdx.x == 0) *out = b.i;
}

// K largest, ties to the lower id (core/math_cpu.cpp:695-707).  Round r picks the
// best element strictly after round r-1's pick in that order.
__global__ void __launch_bounds__(1024) topk_kernel(const float* __restrict__ logits, int V, int K,
                                                    float* __restrict__ vals, int32_t* __restrict__ ids) {
    __shared__ Best sm[32];
    __shared__ Best prev;
    if (threadIdx.x == 0) prev = Best{0.0f, -1};
    __syncthreads();
    for (int r = 0; r < K; ++r) {
        const Best p = prev;
        Best mine{0.0f, -1};
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const Best c{logits[i], i};
            const bool after = p.i < 0 || c.v < p.v || (c.v == p.v && c.i > p.i);
            if (after && better(c, mine)) mine = c;
        }
        const Best b = block_best(mine, sm);
        if (threadIdx.x == 0) {
            vals[r] = b.v;
            ids[r] = b.i;
            prev = b;
        }
        __syncthreads();
    }
}

// Penalties applied once per distinct in-range history token
// (core/math_cpu.cpp:724-753); the first occurrence owns the update.
__global__ void rep_penalty_kernel(float* logits, int V, const int32_t* __restrict__ hist,
                                   int hist_n, float rep, float freq, float pres) {
    const bool use_rep = rep > 0.0f && rep != 1.0f;
    GRID_STRIDE(i, hist_n) {
        const int32_t tok = hist[i];
        if (tok < 0 || tok >= V) continue;
        int count = 0;
        bool first = true;
        for (int j = 0; j < hist_n; ++j) {
            if (hist[j] == tok) {
                if (j < i) { first = false; break; }
                ++count;
            }
        }
        if (!first) continue;
        float l = logits[tok];
        if (use_rep) l = (l > 0.0f) ? l / rep : l * rep;
        if (freq != 0.0f) l -= freq * (float)count;
        if (pres != 0.0f) l -= pres;
        logits[tok] = l;
    }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_add(const float* a, const float* b, float* out, int64_t n) {
    if (n <= 0) return B200_OK;
    B200_REQUIRE(a && b && out, "add: null pointer");
    add_kernel<<<flat_grid(n), 256, 0, stream()>>>(a, b, out, n);
    B200_LAUNCH_CHECK("add_kernel");
    return B200_OK;
}
int b200_add_inplace(float* a, const float* b, int64_t n) { return b200_add(a, b, a, n); }
int b200_add_bias(const float* b, float* y, int64_t rows, int cols) {
    if (rows <= 0 || cols <= 0) return B200_OK;
    B200_REQUIRE(b && y, "add_bias: null pointer");
    add_bias_kernel<<<flat_grid(rows * cols), 256, 0, stream()>>>(b, y, rows * cols, cols);
    B200_LAUNCH_CHECK("add_bias_kernel");
    return B200_OK;
}
int b200_scale_inplace(float* a, float s, int64_t n) {
    if (n <= 0) return B200_OK;
    B200_REQUIRE(a, "scale_inplace: null pointer");
    scale_kernel<<<flat_grid(n), 256, 0, stream()>>>(a, s, n);
    B200_LAUNCH_CHECK("scale_kernel");
    return B200_OK;
}
int b200_zero(float* a, int64_t n) {
    if (n <= 0) return B200_OK;
    B200_REQUIRE(a, "zero: null pointer");
    B200_CUDA(cudaMemsetAsync(a, 0, (size_t)n * 4, stream()));
    return B200_OK;
}
int b200_copy_f32(float* dst, const float* src, int64_t n) {
    if (n <= 0) return B200_OK;
    B200_REQUIRE(dst && src, "copy: null pointer");
    B200_CUDA(cudaMemcpyAsync(dst, src, (size_t)n * 4, cudaMemcpyDeviceToDevice, stream()));
    return B200_OK;
}

int b200_embedding_forward(const int32_t* ids, const float* table, float* out, int64_t ntok, int dim, int vocab) {
    if (ntok <= 0) return B200_OK;
    B200_REQUIRE(ids && table && out && dim > 0 && vocab > 0, "embedding_forward: bad arguments");
    embedding_kernel<false><<<(unsigned)ntok, 256, 0, stream()>>>(ids, table, out, dim, vocab);
    B200_LAUNCH_CHECK("embedding_kernel");
    return B200_OK;
}
int b200_embedding_forward_half(const int32_t* ids, const uint16_t* table, float* out, int64_t ntok, int dim, int vocab) {
    if (ntok <= 0) return B200_OK;
    B200_REQUIRE(ids && table && out && dim > 0 && vocab > 0, "embedding_forward_half: bad arguments");
    embedding_kernel<true><<<(unsigned)ntok, 256, 0, stream()>>>(ids, table, out, dim, vocab);
    B200_LAUNCH_CHECK("embedding_kernel");
    return B200_OK;
}
int b200_rmsnorm_forward(const float* x, const float* weight, float* out, float* rrms, int64_t rows, int dim, float eps) {
    if (rows <= 0) return B200_OK;
    B200_REQUIRE(x && weight && out && dim > 0, "rmsnorm_forward: bad arguments");
    rmsnorm_kernel<<<(unsigned)rows, 256, 0, stream()>>>(x, weight, out, rrms, dim, eps);
    B200_LAUNCH_CHECK("rmsnorm_kernel");
    return B200_OK;
}
int b200_rope_forward_cached(float* q, float* k, const int32_t* pos, const float* inv_freq, int64_t ntok,
                             int n_heads, int n_kv, int head_dim, int rope_type) {
    if (ntok <= 0) return B200_OK;
    B200_REQUIRE(pos && inv_freq && head_dim > 0 && head_dim % 2 == 0, "rope_forward_cached: bad arguments");
    rope_cached_kernel<<<flat_grid(ntok * (head_dim / 2)), 256, 0, stream()>>>(q, k, pos, inv_freq, ntok, n_heads,
                                                                               n_kv, head_dim, rope_type);
    B200_LAUNCH_CHECK("rope_cached_kernel");
    return B200_OK;
}
int b200_swiglu_forward(const float* g, const float* u, float* out, int64_t n) {
    if (n <= 0) return B200_OK;
    B200_REQUIRE(g && u && out, "swiglu_forward: null pointer");
    swiglu_kernel<<<flat_grid(n), 256, 0, stream()>>>(g, u, out, n);
    B200_LAUNCH_CHECK("swiglu_kernel");
    return B200_OK;
}

int b200_argmax_token_device(const float* logits, int V, int32_t* token_dev) {
    B200_REQUIRE(V > 0, "argmax_token: empty vocabulary");
    B200_REQUIRE(logits && token_dev, "argmax_token: null pointer");
    argmax_kernel<<<1, 1024, 0, stream()>>>(logits, V, token_dev);
    B200_LAUNCH_CHECK("argmax_kernel");
    return B200_OK;
}
int b200_argmax_token(const float* logits, int V, int32_t* token_host) {
    B200_REQUIRE(token_host, "argmax_token: null pointer");
    void* ws;
    int rc = workspace(WS_SAMPLE).ensure(256, &ws);
    if (rc) return rc;
    rc = b200_argmax_token_device(logits, V, static_cast<int32_t*>(ws));
    if (rc) return rc;
    B200_CUDA(cudaMemcpyAsync(token_host, ws, 4, cudaMemcpyDeviceToHost, stream()));
    B200_CUDA(cudaStreamSynchronize(stream()));
    return B200_OK;
}
int b200_topk_select(const float* logits, int V, int K, float* out_vals, int32_t* out_ids) {
    B200_REQUIRE(V > 0 && K >= 1 && K <= V, "topk_select: K out of range");
    B200_REQUIRE(logits && out_vals && out_ids, "topk_select: null pointer");
    topk_kernel<<<1, 1024, 0, stream()>>>(logits, V, K, out_vals, out_ids);
    B200_LAUNCH_CHECK("topk_kernel");
    return B200_OK;
}
int b200_apply_rep_penalties(float* logits, int V, const int32_t* hist, int hist_n, float rep, float freq, float pres) {
    if (hist_n <= 0 || V <= 0) return B200_OK;
    const bool use_rep = rep > 0.0f && rep != 1.0f;
    if (!use_rep && freq == 0.0f && pres == 0.0f) return B200_OK;
    B200_REQUIRE(logits && hist, "apply_rep_penalties: null pointer");
    // The reference hands over the history as a HOST array (it stages it itself,
    // cuda/kernels.cu:1279-1308); a device pointer is accepted as well and used in place.
    cudaPointerAttributes at;
    const cudaError_t q = cudaPointerGetAttributes(&at, hist);
    if (q != cudaSuccess) cudaGetLastError();
    const bool on_device = q == cudaSuccess && (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged);
    if (!on_device) {
        void* ws;
        const int rc = workspace(WS_SAMPLE).ensure((size_t)hist_n * 4 + 256, &ws);
        if (rc) return rc;
        B200_CUDA(cudaMemcpyAsync(ws, hist, (size_t)hist_n * 4, cudaMemcpyHostToDevice, stream()));
        hist = static_cast<const int32_t*>(ws);
    }
    rep_penalty_kernel<<<flat_grid(hist_n), 256, 0, stream()>>>(logits, V, hist, hist_n, rep, freq, pres);
    B200_LAUNCH_CHECK("rep_penalty_kernel");
    return B200_OK;
}

}  // extern "C"
