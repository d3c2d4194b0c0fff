// Tensor-core GEMM for the many-token side of the hot path (prefill linears,
// batched decode, the grouped SwiGLU experts of the MoE layer):
//
//     C[rows, N] = A[rows, K] . B[N, K]^T          fp16 operands, fp32 accumulation
//
// on the 5th-generation tensor cores: operand tiles are brought into shared memory
// by 2-D TMA loads (128-byte swizzle), one elected thread issues tcgen05.mma with
// the accumulator in tensor memory, four warps read it back with tcgen05.ld and run
// the epilogue.  The reference reaches the same shapes through cuBLAS GemmEx on an
// fp16 copy of the activations (cuda/kernels.cu:600-633) and one cuBLAS call per
// expert (cuda/moe.cu:731-958).
//
// Grouped form: the rows of A are partitioned into `groups` consecutive ranges
// (offsets[g] .. offsets[g+1], device memory) and range g multiplies rows
// [g*N, (g+1)*N) of B - the expert-sorted token rows of the MoE layer.  The tile
// list is the concatenation of every group's 128-row tiles; a CTA finds its own by
// walking the offsets, so no host synchronisation is needed to size the grid.
//
// One CTA = one 128 x 128 output tile, 192 threads:
//   warp 0      TMA producer (one lane): A tile and B tile(s) of each 64-wide K block
//   warp 1      tensor-memory allocation, MMA issue (one lane), deallocation
//   warps 2..5  epilogue, one 32-row quarter of the accumulator each
// Every mbarrier wait is bounded; when a bound is hit the kernel raises the status
// word, skips its stores, and still releases its tensor memory.
#include <cuda_fp16.h>

#include <map>
#include <mutex>
#include <tuple>

#include "gemm.cuh"
#include "umma.cuh"

namespace b200 {

constexpr int GM_TILE_M = 128, GM_TILE_N = 128, GM_TILE_K = 64;
constexpr int GM_THREADS = 192;
constexpr int GM_STAGE_A = GM_TILE_M * GM_TILE_K * 2;

struct alignas(64) GemmArgs {
    CUtensorMap map_a, map_b, map_b2;   // b2: the "up" matrix of the SwiGLU form
    const int32_t* offsets;             // device [groups + 1], or null: one group [0, M)
    int M, groups, N, K;
    float* c;                           // STORE: fp32 [M, ldc]
    __half* c16;                        // SWIGLU: fp16 [M, ldc]  silu(A.B^T) * (A.B2^T)
    int64_t ldc;
    float scale;
    int* status;
};

template <int EPI>
struct GemmShape {
    static constexpr int UN = EPI == GEMM_EPI_SWIGLU ? 2 * GM_TILE_N : GM_TILE_N;   // MMA N = accumulator columns
    static constexpr int STAGE_B = UN * GM_TILE_K * 2;
    static constexpr int STAGE = GM_STAGE_A + STAGE_B;
    static constexpr int STAGES = EPI == GEMM_EPI_SWIGLU ? 4 : 6;
    static constexpr int SMEM = STAGES * STAGE + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int EPI>
__global__ void __launch_bounds__(GM_THREADS, 1) umma_gemm_kernel(const __grid_constant__ GemmArgs a) {
    using S = GemmShape<EPI>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::STAGES * S::STAGE);
    uint64_t* empty = full + S::STAGES;
    uint64_t* accum = empty + S::STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- which tile: (group, first row, row limit) -------------------------------
    int group = 0, row0 = 0, row_end = a.M;
    {
        int slot = blockIdx.y;
        if (a.offsets) {
            bool found = false;
            int lo = a.offsets[0];
            for (int g = 0; g < a.groups; ++g) {
                const int hi = a.offsets[g + 1];
                const int tiles = (hi - lo + GM_TILE_M - 1) / GM_TILE_M;
                if (slot < tiles) {
                    group = g; row0 = lo + slot * GM_TILE_M; row_end = hi; found = true;
                    break;
                }
                slot -= tiles;
                lo = hi;
            }
            if (!found) return;                       // uniform for the whole CTA
        } else {
            row0 = slot * GM_TILE_M;
            if (row0 >= a.M) return;
        }
    }
    const int n0 = blockIdx.x * GM_TILE_N;            // first output column inside the group
    const int brow0 = group * a.N + n0;               // first row of B
    const int KB = (a.K + GM_TILE_K - 1) / GM_TILE_K;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, S::UN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < KB; ++kb) {
                const int s = kb % S::STAGES;
                if (kb >= S::STAGES && !mbar_wait(&empty[s], ((kb / S::STAGES) - 1) & 1, a.status)) break;
                uint8_t* st = smem + (size_t)s * S::STAGE;
                mbar_expect_tx(&full[s], S::STAGE);
                tma_load_2d(st, &a.map_a, kb * GM_TILE_K, row0, &full[s]);
                tma_load_2d(st + GM_STAGE_A, &a.map_b, kb * GM_TILE_K, brow0, &full[s]);
                if (EPI == GEMM_EPI_SWIGLU)
                    tma_load_2d(st + GM_STAGE_A + GM_TILE_N * GM_TILE_K * 2, &a.map_b2, kb * GM_TILE_K, brow0, &full[s]);
                issued = kb + 1;
            }
            if (issued < KB) {
                // gave up: do not leave with copies of this CTA still landing in shared memory
                for (int kb = max(0, issued - S::STAGES); kb < issued; ++kb)
                    if (!mbar_wait(&full[kb % S::STAGES], (kb / S::STAGES) & 1, a.status)) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(GM_TILE_M, S::UN);
            bool ok = true;
            for (int kb = 0; kb < KB && ok; ++kb) {
                const int s = kb % S::STAGES;
                ok = mbar_wait(&full[s], (kb / S::STAGES) & 1, a.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + (size_t)s * S::STAGE);
                const uint32_t b_addr = a_addr + GM_STAGE_A;
#pragma unroll
                for (int k = 0; k < GM_TILE_K / 16; ++k)
                    umma_f16(tmem, umma_smem_desc(a_addr + k * 32), umma_smem_desc(b_addr + k * 32), idesc,
                             kb > 0 || k > 0);
                umma_commit(&empty[s]);               // the stage is free once these MMAs have read it
            }
            umma_commit(accum);                       // accumulator complete (or as far as we got)
        }
    } else {
        const int q = warp & 3;                       // tensor-memory lane quarter this warp may read
        const int row = row0 + q * 32 + lane;
        bool ok = mbar_wait(accum, 0, a.status);
        tc_fence_after();
        // a failed wait anywhere in the CTA leaves the status word set: skip the stores
        // (decided per warp: tcgen05.ld is a warp-wide instruction)
        ok = __all_sync(0xffffffffu, ok && *reinterpret_cast<volatile int*>(a.status) == 0);
        if (ok) {
            const uint32_t tbase = tmem + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < GM_TILE_N; c0 += 32) {
                float v[32];
                tmem_ld32(tbase + c0, v);
                if (EPI == GEMM_EPI_SWIGLU) {
                    float u[32];
                    tmem_ld32(tbase + GM_TILE_N + c0, u);
                    if (row < row_end) {
                        __half* dst = a.c16 + (int64_t)row * a.ldc + n0 + c0;
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            if (n0 + c0 + i + 1 < a.N) {
                                *reinterpret_cast<__half2*>(dst + i) =
                                    __floats2half2_rn(silu_acc(v[i]) * u[i], silu_acc(v[i + 1]) * u[i + 1]);
                            } else if (n0 + c0 + i < a.N) {
                                dst[i] = __float2half_rn(silu_acc(v[i]) * u[i]);
                            }
                        }
                    }
                } else if (row < row_end) {
                    float* dst = a.c + (int64_t)row * a.ldc + n0 + c0;
                    if (n0 + c0 + 32 <= a.N && (a.ldc & 3) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4*>(dst + i) =
                                make_float4(v[i] * a.scale, v[i + 1] * a.scale, v[i + 2] * a.scale, v[i + 3] * a.scale);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (n0 + c0 + i < a.N) dst[i] = v[i] * a.scale;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, S::UN);
}

// ===========================================================================
// fp32 rows -> fp16 rows (optionally gathered): the A operand
// ===========================================================================
// dst[r, :] = half(src[(row_map ? row_map[r] / div : r), :]), values clamped to the
// fp16 range.  One warp per row, 8 values per lane per step.
__global__ void __launch_bounds__(256) pack_rows_f16_kernel(const float* __restrict__ src, const int32_t* __restrict__ row_map,
                                                           int div, __half* __restrict__ dst, int64_t rows, int K) {
    const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const int64_t sr = row_map ? (int64_t)(row_map[r] / div) : r;
    const float* s = src + sr * K;
    __half* d = dst + r * K;
    for (int k = lane * 8; k < K; k += 256) {
        const float4 a = *reinterpret_cast<const float4*>(s + k);
        const float4 b = *reinterpret_cast<const float4*>(s + k + 4);
        auto cl = [](float v) { return fminf(fmaxf(v, -65504.0f), 65504.0f); };
        __half2 h[4] = {__floats2half2_rn(cl(a.x), cl(a.y)), __floats2half2_rn(cl(a.z), cl(a.w)),
                        __floats2half2_rn(cl(b.x), cl(b.y)), __floats2half2_rn(cl(b.z), cl(b.w))};
        *reinterpret_cast<uint4*>(d + k) = *reinterpret_cast<uint4*>(h);
    }
}

int pack_rows_f16(const float* src, const int32_t* row_map, int div, __half* dst, int64_t rows, int K) {
    B200_REQUIRE(src && dst && rows >= 0 && K > 0 && K % 8 == 0, "pack_rows_f16: K must be a positive multiple of 8");
    B200_REQUIRE((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0,
                 "pack_rows_f16: buffers must be 16-byte aligned");
    if (rows == 0) return B200_OK;
    pack_rows_f16_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream()>>>(src, row_map, div > 0 ? div : 1, dst, rows, K);
    B200_LAUNCH_CHECK("pack_rows_f16_kernel");
    return B200_OK;
}

// ===========================================================================
// host side
// ===========================================================================
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int make_tile_map(CUtensorMap* out, const void* base, int64_t rows, int64_t K, int box_rows) {
    B200_REQUIRE(base && rows > 0 && K > 0 && K % 8 == 0, "tile map: K must be a positive multiple of 8");
    B200_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tile map: base must be 16-byte aligned");
    B200_REQUIRE(box_rows >= 8 && box_rows <= 256, "tile map: bad box");
    typedef std::tuple<const void*, int64_t, int64_t, int> Key;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const Key key(base, rows, K, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return B200_OK;
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(B200_ECUDA, "tile map: the driver does not export cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)GM_TILE_K, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200_ECUDA, "tile map: cuTensorMapEncodeTiled failed with %d", (int)r);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return B200_OK;
}

template <int EPI>
static int launch_gemm(const GemmArgs& a) {
    using S = GemmShape<EPI>;
    auto kern = umma_gemm_kernel<EPI>;
    static bool configured = false;
    if (!configured) {
        B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM));
        configured = true;
    }
    const int m_slots = (a.M + GM_TILE_M - 1) / GM_TILE_M + (a.offsets ? a.groups : 0);
    dim3 grid((a.N + GM_TILE_N - 1) / GM_TILE_N, m_slots);
    B200_REQUIRE(m_slots <= 65535, "umma_gemm: too many row tiles (%d)", m_slots);
    kern<<<grid, GM_THREADS, S::SMEM, stream()>>>(a);
    B200_LAUNCH_CHECK("umma_gemm_kernel");
    return B200_OK;
}

// A [a_rows, K] fp16; B (and B2) [b_rows, K] fp16 with b_rows = groups * N.
// offsets: device [groups + 1] or null (then groups must be 1 and all M rows form it).
int umma_gemm(int epi, const __half* A, int64_t a_rows, const __half* B, const __half* B2, int64_t b_rows,
              const int32_t* offsets, int groups, int M, int N, int K, float* c, __half* c16, int64_t ldc, float scale) {
    if (M <= 0 || N <= 0) return B200_OK;
    B200_REQUIRE(A && B && K > 0 && K % 8 == 0, "umma_gemm: K must be a positive multiple of 8");
    B200_REQUIRE(groups >= 1 && (offsets || groups == 1), "umma_gemm: groups need a device offsets array");
    B200_REQUIRE(b_rows >= (int64_t)groups * N && a_rows >= M, "umma_gemm: operand shapes do not cover the groups");
    GemmArgs a;
    int rc = make_tile_map(&a.map_a, A, a_rows, K, GM_TILE_M);
    if (rc) return rc;
    rc = make_tile_map(&a.map_b, B, b_rows, K, GM_TILE_N);
    if (rc) return rc;
    a.map_b2 = a.map_b;
    if (epi == GEMM_EPI_SWIGLU) {
        B200_REQUIRE(B2 && c16 && ldc % 2 == 0, "umma_gemm: the SwiGLU form needs the second matrix and an fp16 output");
        rc = make_tile_map(&a.map_b2, B2, b_rows, K, GM_TILE_N);
        if (rc) return rc;
    } else {
        B200_REQUIRE(c, "umma_gemm: null output");
    }
    a.offsets = offsets; a.M = M; a.groups = groups; a.N = N; a.K = K;
    a.c = c; a.c16 = c16; a.ldc = ldc; a.scale = scale;
    a.status = stream_status_ptr();
    B200_REQUIRE(a.status, "umma_gemm: status word allocation failed");
    return epi == GEMM_EPI_SWIGLU ? launch_gemm<GEMM_EPI_SWIGLU>(a) : launch_gemm<GEMM_EPI_STORE>(a);
}

}  // namespace b200
