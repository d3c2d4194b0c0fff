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
// list is the concatenation of every group's 128-row tiles; a CTA finds a tile by
// walking the offsets, so no host synchronisation is needed to size the grid.
//
// Persistent kernel: one CTA per SM walks the 128 x 128 output tiles t = blockIdx.x,
// + gridDim.x, ...  The operand ring runs on across tile boundaries and there are
// two accumulators in tensor memory, so the epilogue of one tile overlaps the main
// loop of the next.
//   warp 0      TMA producer (one lane): A tile and B tile(s) of each 64-wide K block
//   warp 1      tensor-memory allocation, MMA issue (one lane), deallocation
//   warps 2..5  epilogue, one 32-row quarter of the accumulator each
// Every mbarrier wait is bounded; when a bound is hit the kernel raises the status
// word, the role that hit it stops, the others run into their own bounds, nothing
// more is stored, and the tensor memory is still released.
#include <cuda_fp16.h>

#include <map>
#include <mutex>
#include <tuple>

#include "gemm.cuh"
#include "umma.cuh"

namespace b200 {

constexpr int GM_TILE_M = 128, GM_TILE_N = 128, GM_TILE_K = 64;
// Third epilogue, chosen by the launchers for large store-form problems: the store form on
// 256-column tiles (one N = 256 MMA per K step over two 128-row boxes of B).  With
// cta_group::1 both MMA operands come out of shared memory, so a 128 x 128 x 16 MMA moves
// 8 KB per 32 tensor-core cycles and a 128 x 256 x 16 one 12 KB per 64: the wide tile lifts
// the operand-bandwidth cap from about half to about two thirds of the tensor peak, and A is
// re-streamed from L2 half as often.
constexpr int GEMM_EPI_STORE_WIDE = 2;
constexpr int GM_THREADS = 192;
constexpr int GM_STAGE_A = GM_TILE_M * GM_TILE_K * 2;
// Per epilogue warp: a 32 x 32 fp32 block (rows padded to 33) through which the
// accumulator rows a lane holds are turned into stores of whole 128-byte lines.
constexpr int GM_EPI_LD = 33;
constexpr int GM_EPI_SCRATCH = 4 * 32 * GM_EPI_LD * 4;
// Row-slot table of the grouped form (see gemm_build_slots).
constexpr int GM_MAX_SLOTS = 448;
constexpr int GM_SLOT_TABLE = (1 + 3 * GM_MAX_SLOTS) * 4 + 12;

struct alignas(64) GemmArgs {
    CUtensorMap map_a, map_b, map_b2;   // b2: the "up" matrix of the SwiGLU form
    const int32_t* offsets;             // device [groups + 1], or null: one group [0, M)
    const int32_t* group_map;           // device [groups]: which N-row block of B a group uses; null = its own index
    int M, groups, N, K;
    int m_slots, n_tiles;               // tile grid: slots along the rows (an upper bound when grouped) x column tiles
    int tile_n;                         // output columns per tile: 128, or 256 (wide store form)
    int tile_m;                         // rows of A per slot: 128, or 256 = two accumulator halves sharing one B tile
    float* c;                           // STORE: fp32 [M, ldc]
    // STORE, grouped, optional: device [groups] of bases that replace `c` for a group's rows:
    // row r of group g is stored at group_c[g] + r * ldc (r counted like the rows of A, so a
    // caller that wants the group's first row at p passes p - offsets[g] * ldc).  The
    // targets may be peer memory (plain stores).
    float* const* group_c;
    __half* c16;                        // SWIGLU: fp16 [M, ldc]  silu(A.B^T) * (A.B2^T)
    int64_t ldc;
    float scale;
    int* status;
    // split K (packed-weight store form with few tiles): the tile list is repeated k_splits
    // times, repetition s covers K steps [s * kb_split, (s + 1) * kb_split) and stores its
    // partial product at c + s * split_stride; a second kernel adds the partials in order
    int k_splits, kb_split;
    int64_t split_stride;
    bool allow_split_k;                 // host only: false keeps one K range whatever the tile count
};

template <int EPI>
struct GemmShape {
    static constexpr int UN = EPI == GEMM_EPI_STORE ? GM_TILE_N : 2 * GM_TILE_N;   // MMA N = accumulator columns
    static constexpr int TN = EPI == GEMM_EPI_STORE_WIDE ? 2 * GM_TILE_N : GM_TILE_N;   // output columns of a tile
    static constexpr int STAGE_B = UN * GM_TILE_K * 2;
    static constexpr int STAGE = GM_STAGE_A + STAGE_B;
    static constexpr int STAGES = EPI == GEMM_EPI_STORE ? 6 : 4;
    static constexpr int SMEM = STAGES * STAGE + GM_EPI_SCRATCH + 1024 /*alignment slack*/ + 256 /*barriers*/ + GM_SLOT_TABLE;
};

// One tile of the walk.
struct GemmTile {
    int group, row0, row_end, n0, brow0;
    int split;                          // which K range (0 unless the launch splits K)
};

// Grouped form: row slot -> (group, first row, end of the group), built once per CTA in
// shared memory so that every role finds a tile with one load instead of a walk over the
// offsets (with K of a few hundred a tile lasts a few microseconds, and a walk over 64
// groups costs about two).  tab[0] = slots in use, then 3 ints per slot.

// All threads of the CTA; `scan` is scratch for 2 * (groups + 1) ints.  Leaves tab[0] = -1
// (callers then walk the offsets) when there are more groups or slots than the table holds.
__device__ __noinline__ void gemm_build_slots(const GemmArgs& a, int* tab, int* scan) {
    if (!a.offsets) return;
    // (m_slots is the host's upper bound from the row count; lists with gaps between their
    // groups hold far fewer tiles, so the bound only decides for lists the scan cannot hold)
    const bool fits = a.groups <= 256;
    if (!fits) {
        if (threadIdx.x == 0) tab[0] = -1;
        return;
    }
    int* cnt = scan;                 // [groups]
    int* base = scan + a.groups;     // [groups + 1]
    // a group mapped to a negative block is a gap between groups: its rows are skipped
    for (int g = threadIdx.x; g < a.groups; g += blockDim.x)
        cnt[g] = (a.group_map && a.group_map[g] < 0) ? 0 : (a.offsets[g + 1] - a.offsets[g] + a.tile_m - 1) / a.tile_m;
    __syncthreads();
    if (threadIdx.x < 32) {
        const int per = (a.groups + 31) >> 5, g0 = threadIdx.x * per;
        int sum = 0;
        for (int i = 0; i < per; ++i)
            if (g0 + i < a.groups) sum += cnt[g0 + i];
        int incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if ((int)threadIdx.x >= o) incl += up;
        }
        int run = incl - sum;
        for (int i = 0; i < per; ++i)
            if (g0 + i < a.groups) {
                base[g0 + i] = run;
                run += cnt[g0 + i];
            }
        // more row tiles than slots: keep the first slot of every group instead (tab[0] = -2,
        // tab[1 + g] = first slot of group g, tab[1 + groups] = slots in all) and let the roles
        // find a slot's group by bisection
        if (threadIdx.x == 31) {
            tab[0] = incl <= GM_MAX_SLOTS ? incl : -2;
            base[a.groups] = incl;
        }
    }
    __syncthreads();
    if (tab[0] == -2) {
        for (int g = threadIdx.x; g <= a.groups; g += blockDim.x) tab[1 + g] = base[g];
        return;
    }
    for (int g = threadIdx.x; g < a.groups; g += blockDim.x) {
        const int lo = a.offsets[g], hi = a.offsets[g + 1];
        for (int i = 0; i < cnt[g]; ++i) {
            const int s = base[g] + i;
            if (s < GM_MAX_SLOTS) {
                tab[1 + 3 * s] = g;
                tab[2 + 3 * s] = lo + i * a.tile_m;
                tab[3 + 3 * s] = hi;
            }
        }
    }
}

// The walk over the offsets for group lists the table does not hold.
__device__ __noinline__ int4 gemm_slot_walk(const int32_t* offsets, const int32_t* group_map, int groups, int tile_m,
                                            int slot) {
    int lo = offsets[0];
    for (int g = 0; g < groups; ++g) {
        const int hi = offsets[g + 1];
        const int tiles = (group_map && group_map[g] < 0) ? 0 : (hi - lo + tile_m - 1) / tile_m;
        if (slot < tiles) return make_int4(1, g, lo + slot * tile_m, hi);
        slot -= tiles;
        lo = hi;
    }
    return make_int4(0, 0, 0, 0);
}

// Tile t of the list -> coordinates; false when the slot lies past the last row tile
// (the grouped list is sized by an upper bound).
__device__ __forceinline__ bool gemm_tile_at(const GemmArgs& a, const int* tab, int t, GemmTile& w) {
    w.split = 0;
    if (a.k_splits > 1) {
        w.split = t % a.k_splits;
        t /= a.k_splits;
    }
    const int slot = t / a.n_tiles;
    w.n0 = (t - slot * a.n_tiles) * a.tile_n;
    w.group = 0; w.row0 = 0; w.row_end = a.M;
    bool found;
    if (!a.offsets) {
        w.row0 = slot * a.tile_m;
        found = w.row0 < a.M;
    } else if (tab[0] >= 0) {
        found = slot < tab[0];
        if (found) { w.group = tab[1 + 3 * slot]; w.row0 = tab[2 + 3 * slot]; w.row_end = tab[3 + 3 * slot]; }
    } else if (tab[0] == -2) {
        const int* first = tab + 1;
        found = slot < first[a.groups];
        if (found) {
            int lo = 0, hi = a.groups;               // the last group whose first slot is <= slot
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (first[mid] <= slot) lo = mid; else hi = mid;
            }
            // groups without tiles share their first slot with the next one: lo is the last of
            // such a run, which is the one that owns the slot
            w.group = lo;
            w.row0 = a.offsets[lo] + (slot - first[lo]) * a.tile_m;
            w.row_end = a.offsets[lo + 1];
        }
    } else {
        const int4 r = gemm_slot_walk(a.offsets, a.group_map, a.groups, a.tile_m, slot);
        found = r.x != 0;
        if (found) { w.group = r.y; w.row0 = r.z; w.row_end = r.w; }
    }
    w.brow0 = (a.group_map && found ? a.group_map[w.group] : w.group) * a.N + w.n0;
    return found;
}

// silu for the SwiGLU epilogue, whose result is rounded to fp16 (2^-11) right away: the
// fast exponential and reciprocal (a few fp32 ulp) are invisible at that precision and
// cost a fifth of the accurate forms, which matters because this epilogue (65536
// activations per tile on four warps) is not hidden behind a second accumulator set.
__device__ __forceinline__ float silu_fast(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

// Epilogue of one 128 x 128 tile out of the accumulator at `tacc`, run by the four
// warps whose index modulo 4 selects the 32 accumulator rows (tensor-memory lanes) a
// warp may read.
template <int EPI>
__device__ __forceinline__ void gemm_epilogue(const GemmArgs& a, uint32_t tacc, int warp, int lane, const GemmTile& w,
                                              float* scratch) {
    const int q = warp & 3;
    float* stg = scratch + q * 32 * GM_EPI_LD;
    const int row = w.row0 + q * 32 + lane;
    const int row_end = w.row_end, n0 = w.n0;
    const uint32_t tbase = tacc + ((uint32_t)(q * 32) << 16);
    float* const cbase = (EPI != GEMM_EPI_SWIGLU && a.group_c) ? a.group_c[w.group] : a.c + w.split * a.split_stride;
#pragma unroll 1
    for (int c0 = 0; c0 < GemmShape<EPI>::TN; c0 += 32) {
        float v[32];
        tmem_ld32(tbase + c0, v);
        if (EPI == GEMM_EPI_SWIGLU) {
            float u[32];
            tmem_ld32(tbase + GM_TILE_N + c0, u);
            if (n0 + c0 + 32 <= a.N && (a.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(a.c16) & 7) == 0) {
                // as the store form below: through the warp's shared block, so that eight
                // lanes write one row's 64 bytes and an instruction covers four rows
#pragma unroll
                for (int i = 0; i < 32; ++i) stg[lane * GM_EPI_LD + i] = silu_fast(v[i]) * u[i];
                __syncwarp();
                const int cq = 4 * (lane & 7);
#pragma unroll
                for (int itr = 0; itr < 8; ++itr) {
                    const int r = itr * 4 + (lane >> 3);
                    const int grow = w.row0 + q * 32 + r;
                    const float* sp = stg + r * GM_EPI_LD + cq;
                    if (grow < row_end) {
                        const __half2 h01 = __floats2half2_rn(sp[0], sp[1]), h23 = __floats2half2_rn(sp[2], sp[3]);
                        uint2 pk;
                        pk.x = *reinterpret_cast<const uint32_t*>(&h01);
                        pk.y = *reinterpret_cast<const uint32_t*>(&h23);
                        *reinterpret_cast<uint2*>(a.c16 + (int64_t)grow * a.ldc + n0 + c0 + cq) = pk;
                    }
                }
                __syncwarp();
            } else if (row < row_end) {
                __half* dst = a.c16 + (int64_t)row * a.ldc + n0 + c0;
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    if (n0 + c0 + i + 1 < a.N) {
                        *reinterpret_cast<__half2*>(dst + i) =
                            __floats2half2_rn(silu_fast(v[i]) * u[i], silu_fast(v[i + 1]) * u[i + 1]);
                    } else if (n0 + c0 + i < a.N) {
                        dst[i] = __float2half_rn(silu_fast(v[i]) * u[i]);
                    }
                }
            }
        } else if (n0 + c0 + 32 <= a.N && (a.ldc & 3) == 0) {
            // lane = row in registers -> shared block -> eight lanes per row write one
            // 128-byte line, four rows per instruction
#pragma unroll
            for (int i = 0; i < 32; ++i) stg[lane * GM_EPI_LD + i] = v[i] * a.scale;
            __syncwarp();
            const int cq = 4 * (lane & 7);
#pragma unroll
            for (int itr = 0; itr < 8; ++itr) {
                const int r = itr * 4 + (lane >> 3);
                const int grow = w.row0 + q * 32 + r;
                const float* sp = stg + r * GM_EPI_LD + cq;
                if (grow < row_end)
                    *reinterpret_cast<float4*>(cbase + (int64_t)grow * a.ldc + n0 + c0 + cq) =
                        make_float4(sp[0], sp[1], sp[2], sp[3]);
            }
            __syncwarp();
        } else if (row < row_end) {
            float* dst = cbase + (int64_t)row * a.ldc + n0 + c0;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (n0 + c0 + i < a.N) dst[i] = v[i] * a.scale;
        }
    }
}

// The epilogue warps' loop over this CTA's tiles: wait for the accumulator, drain it,
// hand it back to the MMA warp.  Stops storing as soon as the status word is raised.
// ACC accumulator sets of HALVES x UN columns each; half h holds rows row0 + 128 h ...
template <int EPI, int UN, int ACC, int HALVES>
__device__ __forceinline__ void gemm_epilogue_loop(const GemmArgs& a, uint32_t tmem, uint64_t* acc_full, uint64_t* acc_empty,
                                                   int warp, int lane, int total, float* scratch, const int* tab) {
    uint32_t ti = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x) {
        GemmTile w;
        if (!gemm_tile_at(a, tab, t, w)) continue;
        const int as = ti % ACC;
        bool ok = mbar_wait(&acc_full[as], (ti / ACC) & 1, a.status);
        ok = __all_sync(0xffffffffu, ok && *reinterpret_cast<volatile int*>(a.status) == 0);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
            if (w.row0 + GM_TILE_M * h < w.row_end) {
                GemmTile wh = w;
                wh.row0 += GM_TILE_M * h;
                gemm_epilogue<EPI>(a, tmem + as * (HALVES * UN) + h * UN, warp, lane, wh, scratch);
            }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[as]);
        ++ti;
    }
}

template <int EPI>
__global__ void __launch_bounds__(GM_THREADS, 1) umma_gemm_kernel(const __grid_constant__ GemmArgs a) {
    using S = GemmShape<EPI>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float* epi_scratch = reinterpret_cast<float*>(smem + S::STAGES * S::STAGE);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::STAGES * S::STAGE + GM_EPI_SCRATCH);
    uint64_t* empty = full + S::STAGES;
    uint64_t* acc_full = empty + S::STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    int* tab = reinterpret_cast<int*>(smem + S::STAGES * S::STAGE + GM_EPI_SCRATCH + 256);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total = a.m_slots * a.n_tiles;
    const int KB = (a.K + GM_TILE_K - 1) / GM_TILE_K;
    gemm_build_slots(a, tab, reinterpret_cast<int*>(epi_scratch));

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * S::UN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                GemmTile w;
                if (!gemm_tile_at(a, tab, t, w)) continue;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % S::STAGES;
                    if (it >= S::STAGES) ok = mbar_wait(&empty[s], ((it / S::STAGES) - 1) & 1, a.status);
                    if (!ok) break;
                    uint8_t* st = smem + (size_t)s * S::STAGE;
                    mbar_expect_tx(&full[s], S::STAGE);
                    tma_load_2d(st, &a.map_a, kb * GM_TILE_K, w.row0, &full[s]);
                    tma_load_2d(st + GM_STAGE_A, &a.map_b, kb * GM_TILE_K, w.brow0, &full[s]);
                    if (EPI == GEMM_EPI_SWIGLU)
                        tma_load_2d(st + GM_STAGE_A + GM_TILE_N * GM_TILE_K * 2, &a.map_b2, kb * GM_TILE_K, w.brow0,
                                    &full[s]);
                    if (EPI == GEMM_EPI_STORE_WIDE)
                        tma_load_2d(st + GM_STAGE_A + GM_TILE_N * GM_TILE_K * 2, &a.map_b, kb * GM_TILE_K,
                                    w.brow0 + GM_TILE_N, &full[s]);
                }
            }
            if (!ok) {
                // gave up: do not leave with copies of this CTA still landing in shared memory
                for (uint32_t j = it > S::STAGES ? it - S::STAGES : 0; j < it; ++j)
                    if (!mbar_wait(&full[j % S::STAGES], (j / S::STAGES) & 1, a.status)) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(GM_TILE_M, S::UN);
            uint32_t it = 0, ti = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                GemmTile w;
                if (!gemm_tile_at(a, tab, t, w)) continue;
                const int as = ti & 1;
                if (ti >= 2) ok = mbar_wait(&acc_empty[as], ((ti >> 1) - 1) & 1, a.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tacc = tmem + as * S::UN;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % S::STAGES;
                    ok = mbar_wait(&full[s], (it / S::STAGES) & 1, a.status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + (size_t)s * S::STAGE);
                    const uint32_t b_addr = a_addr + GM_STAGE_A;
#pragma unroll
                    for (int k = 0; k < GM_TILE_K / 16; ++k)
                        umma_f16(tacc, umma_smem_desc(a_addr + k * 32), umma_smem_desc(b_addr + k * 32), idesc,
                                 kb > 0 || k > 0);
                    umma_commit(&empty[s]);           // the stage is free once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[as]);           // accumulator complete
                ++ti;
            }
        }
    } else {
        gemm_epilogue_loop<EPI, S::UN, 2, 1>(a, tmem, acc_full, acc_empty, warp, lane, total, epi_scratch, tab);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 2 * S::UN);
}

// ===========================================================================
// Packed weights: dequantise inside the GEMM
// ===========================================================================
// Same tiling, but B arrives in its packed form: per 256 weights of K (8 blocks of
// the 32-weight kinds, one Q4_K super-block) a row contributes a fixed number of
// bytes (144 / 160 / 272 / 144), which one 2-D TMA box brings in for all rows of the
// tile.  Eight warps expand it, 64 weights of K per row and step, to fp16 - the
// value the reference's CPU path multiplies with, its dequantised weight rounded to
// fp16 (core/ops.cpp:313-336, :392), to within one fp16 ulp - and store the result in
// the swizzled K-major layout the MMA reads.  HBM sees the packed bytes only.
//
//   warp 0       TMA: A tile per 64 of K, packed B per 256 of K
//   warps 6..13  packed B (shared) -> fp16 B tile (shared, 2 buffers)
//   warp 1       MMA when an A stage and a B tile are both ready
//   warps 2..5   epilogue
template <int KIND>
struct PackedShape {
    static constexpr int SBB = 8 * (KIND == 3 ? 18 : q_block_bytes(KIND));   // bytes per row per 256 of K
};

template <int EPI, int KIND>
struct GemmQShape {
    static constexpr int UN = GemmShape<EPI>::UN;
    static constexpr int SBB = PackedShape<KIND>::SBB;
    static constexpr int B16 = UN * GM_TILE_K * 2;                  // one fp16 B tile
    static constexpr int PACKED = UN * SBB;                         // one packed stage
    // fp16 B tiles: enough of them that the expanding warps run ahead of the MMA rather
    // than in lock-step with it (a hand-off costs a few hundred cycles either way)
    // A CTA owns 256 rows of A: two 128-row accumulator halves are fed by the same
    // expanded B tile, which halves the expansion work per flop.  With 128 accumulator
    // columns per half there is room for two sets (epilogue under the next main loop);
    // the SwiGLU form (256 columns per half) has one.
    static constexpr int A_STAGE = 2 * GM_STAGE_A;
    static constexpr int SA = UN == 128 ? 3 : 2, SB = UN == 128 ? 3 : 2, ACC = UN == 128 ? 2 : 1;
    static constexpr int FIXED = SA * A_STAGE + SB * B16 + GM_EPI_SCRATCH + 1024 + 256 + GM_SLOT_TABLE;
    // packed stages: as many as fit (up to 4) - with few rows of A the kernel is a pure
    // weight stream and needs tens of KB in flight per SM to keep HBM busy
    static constexpr int ROOM = (227 * 1024 - FIXED) / PACKED;
    static constexpr int SP = ROOM >= 4 ? 4 : (ROOM >= 1 ? ROOM : 1);
    static_assert(FIXED + PACKED <= 227 * 1024, "the stages do not fit the shared memory of an SM");
    static constexpr int SMEM = FIXED + SP * PACKED;
};

// Half-precision expansion of packed weights, two values per instruction.  A byte
// b OR-ed into the mantissa of 0x6400 is the fp16 number 1024 + b, so small integers
// become fp16 without a conversion instruction; __byte_perm interleaves two payload
// bytes with two 0x64 bytes into one half2.
__device__ __forceinline__ __half2 magic_pair(uint32_t bytes, uint32_t sel) {
    const uint32_t v = __byte_perm(bytes, 0x64646464u, sel);
    return *reinterpret_cast<const __half2*>(&v);
}
constexpr uint32_t SEL_01 = 0x5140, SEL_23 = 0x5342;   // (byte0, byte1) / (byte2, byte3) of the first operand

// 32 of the 64 weights of K block j of a row (segment of 256 weights at `seg`):
// hh = 0 the first 32 of the block, hh = 1 the last 32.  Written as four 16-byte
// chunks of row r of the swizzled fp16 tile.  Arithmetic in fp16 FMAs:
//   Q4_0  (q - 8) * d,  Q8_0  q * d       exact (one rounding of an exact product)
//   Q4_1  q * d + m                        one rounding
//   Q4_K  (q * sc) * d - fp16(m * dmin)    q * sc exact; the min term rounded first
// against fp16(fp32 value) of the materialising dequantiser: equal for Q4_0 / Q8_0,
// within one fp16 ulp otherwise.
template <int KIND>
__device__ __forceinline__ void dequant_half_block(const uint8_t* seg, int j, int hh, uint8_t* tile, int r) {
    uint8_t* rowp = tile + (size_t)(r >> 3) * 1024 + (size_t)(r & 7) * 128;
    const int sw = r & 7;
    __half2 out[16];
    if (KIND == 3) {
        const uint4 hdr = *reinterpret_cast<const uint4*>(seg);
        int s, m;
        q4k_scale_min_regs(2 * j + hh, hdr.y, hdr.z, hdr.w, s, m);
        const __half d = __ushort_as_half((unsigned short)(hdr.x & 0xFFFF));
        const float dmin = half_bits_to_float((uint16_t)(hdr.x >> 16));
        const __half2 sc2 = __half2half2(__int2half_rn(s));
        const __half2 nsc = __half2half2(__int2half_rn(-1024 * s));          // exact: |1024 * s| <= 64512
        const __half2 d2 = __half2half2(d);
        const __half2 nm = __half2half2(__float2half_rn(-__fmul_rn(dmin, (float)m)));
        const uint4 q0 = *reinterpret_cast<const uint4*>(seg + 16 + 32 * j);
        const uint4 q1 = *reinterpret_cast<const uint4*>(seg + 32 + 32 * j);
        const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t x = (words[i] >> (4 * hh)) & 0x0F0F0F0Fu;
            const __half2 a = __hfma2(magic_pair(x, SEL_01), sc2, nsc);      // q * sc, exact
            const __half2 b = __hfma2(magic_pair(x, SEL_23), sc2, nsc);
            out[2 * i] = __hfma2(a, d2, nm);
            out[2 * i + 1] = __hfma2(b, d2, nm);
        }
    } else if (KIND == 2) {
        const uint16_t* blk = reinterpret_cast<const uint16_t*>(seg + (2 * j + hh) * 34);
        const __half2 d2 = __half2half2(__ushort_as_half(blk[0]));
        const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480));   // 1152 = 1024 + 128
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t x = (uint32_t)blk[1 + i] ^ 0x8080u;              // int8 + 128 as unsigned bytes
            out[i] = __hmul2(__hsub2(magic_pair(x, SEL_01), bias), d2);
        }
    } else {
        const int bb = KIND == 0 ? 18 : 20;
        const uint16_t* blk = reinterpret_cast<const uint16_t*>(seg + (2 * j + hh) * bb);
        const __half2 d2 = __half2half2(__ushort_as_half(blk[0]));
        const __half2 m2 = KIND == 1 ? __half2half2(__ushort_as_half(blk[1])) : __half2half2(__ushort_as_half(0));
        const uint16_t* qs = blk + (KIND == 0 ? 1 : 2);
        const __half2 off = __half2half2(__ushort_as_half((unsigned short)(KIND == 0 ? 0x6408 : 0x6400)));  // 1032 / 1024
        // byte i: low nibble = weight i, high nibble = weight 16 + i
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t p = qs[i];
            const __half2 lo = __hsub2(magic_pair(p & 0x0F0Fu, SEL_01), off);
            const __half2 hi = __hsub2(magic_pair((p >> 4) & 0x0F0Fu, SEL_01), off);
            out[i] = KIND == 0 ? __hmul2(lo, d2) : __hfma2(lo, d2, m2);
            out[8 + i] = KIND == 0 ? __hmul2(hi, d2) : __hfma2(hi, d2, m2);
        }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c)
        *reinterpret_cast<uint4*>(rowp + (((4 * hh + c) ^ sw) << 4)) = *reinterpret_cast<const uint4*>(&out[4 * c]);
}


constexpr int GQ_EXPAND_WARPS = 8;
constexpr int GQ_FIRST_EXPAND = 6;                 // warps 0, 1: TMA, MMA; 2..5: epilogue; 6..13: expansion
constexpr int GQ_THREADS = (GQ_FIRST_EXPAND + GQ_EXPAND_WARPS) * 32;

template <int EPI, int KIND>
__global__ void __launch_bounds__(GQ_THREADS, 1) umma_gemm_q_kernel(const __grid_constant__ GemmArgs a) {
    using S = GemmQShape<EPI, KIND>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sm_a = smem;
    uint8_t* sm_b = sm_a + S::SA * S::A_STAGE;
    uint8_t* sm_p = sm_b + S::SB * S::B16;
    float* epi_scratch = reinterpret_cast<float*>(sm_p + S::SP * S::PACKED);
    uint64_t* a_full = reinterpret_cast<uint64_t*>(sm_p + S::SP * S::PACKED + GM_EPI_SCRATCH);
    uint64_t* a_empty = a_full + S::SA;
    uint64_t* b_full = a_empty + S::SA;
    uint64_t* b_empty = b_full + S::SB;
    uint64_t* p_full = b_empty + S::SB;
    uint64_t* p_empty = p_full + 4;
    uint64_t* acc_full = p_empty + 4;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    int* tab = reinterpret_cast<int*>(sm_p + S::SP * S::PACKED + GM_EPI_SCRATCH + 256);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total = a.m_slots * a.n_tiles * a.k_splits;
    const int KB_ALL = a.K / GM_TILE_K;               // K % 256 == 0 (host)
    gemm_build_slots(a, tab, reinterpret_cast<int*>(epi_scratch));

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::SA; ++s) { mbar_init(&a_full[s], 1); mbar_init(&a_empty[s], 1); }
        for (int s = 0; s < S::SB; ++s) { mbar_init(&b_full[s], GQ_EXPAND_WARPS); mbar_init(&b_empty[s], 1); }
        for (int s = 0; s < S::SP; ++s) { mbar_init(&p_full[s], 1); mbar_init(&p_empty[s], GQ_EXPAND_WARPS); }
        for (int s = 0; s < S::ACC; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 4); }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, S::ACC * 2 * S::UN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0, sbi = 0;                 // K blocks and packed super-blocks issued so far
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                GemmTile w;
                if (!gemm_tile_at(a, tab, t, w)) continue;
                const int kb0 = w.split * a.kb_split, kb1 = min(KB_ALL, kb0 + a.kb_split);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    if ((kb & 3) == 0) {
                        const int p = sbi % S::SP;
                        if (sbi >= S::SP) ok = mbar_wait(&p_empty[p], ((sbi / S::SP) - 1) & 1, a.status);
                        if (!ok) break;
                        uint8_t* dst = sm_p + (size_t)p * S::PACKED;
                        mbar_expect_tx(&p_full[p], S::PACKED);
                        tma_load_2d(dst, &a.map_b, (kb >> 2) * (S::SBB / 4), w.brow0, &p_full[p]);
                        if (EPI == GEMM_EPI_SWIGLU)
                            tma_load_2d(dst + GM_TILE_N * S::SBB, &a.map_b2, (kb >> 2) * (S::SBB / 4), w.brow0, &p_full[p]);
                        if (EPI == GEMM_EPI_STORE_WIDE)
                            tma_load_2d(dst + GM_TILE_N * S::SBB, &a.map_b, (kb >> 2) * (S::SBB / 4), w.brow0 + GM_TILE_N,
                                        &p_full[p]);
                        ++sbi;
                    }
                    const int s = it % S::SA;
                    if (it >= S::SA) ok = mbar_wait(&a_empty[s], ((it / S::SA) - 1) & 1, a.status);
                    if (!ok) break;
                    const bool two = w.row0 + GM_TILE_M < w.row_end;      // second half holds rows of this tile
                    mbar_expect_tx(&a_full[s], two ? S::A_STAGE : GM_STAGE_A);
                    tma_load_2d(sm_a + (size_t)s * S::A_STAGE, &a.map_a, kb * GM_TILE_K, w.row0, &a_full[s]);
                    if (two)
                        tma_load_2d(sm_a + (size_t)s * S::A_STAGE + GM_STAGE_A, &a.map_a, kb * GM_TILE_K,
                                    w.row0 + GM_TILE_M, &a_full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(GM_TILE_M, S::UN);
            uint32_t it = 0, ti = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                GemmTile w;
                if (!gemm_tile_at(a, tab, t, w)) continue;
                const int as = ti % S::ACC;
                if (ti >= S::ACC) ok = mbar_wait(&acc_empty[as], ((ti / S::ACC) - 1) & 1, a.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tacc = tmem + as * (2 * S::UN);
                const bool two = w.row0 + GM_TILE_M < w.row_end;
                const int kb0 = w.split * a.kb_split, kb1 = min(KB_ALL, kb0 + a.kb_split);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % S::SA, b = it % S::SB;
                    ok = mbar_wait(&a_full[s], (it / S::SA) & 1, a.status) &&
                         mbar_wait(&b_full[b], (it / S::SB) & 1, a.status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(sm_a + (size_t)s * S::A_STAGE);
                    const uint32_t b_addr = smem_u32(sm_b + (size_t)b * S::B16);
#pragma unroll
                    for (int k = 0; k < GM_TILE_K / 16; ++k)
                        umma_f16(tacc, umma_smem_desc(a_addr + k * 32), umma_smem_desc(b_addr + k * 32), idesc,
                                 kb > kb0 || k > 0);
                    if (two) {
#pragma unroll
                        for (int k = 0; k < GM_TILE_K / 16; ++k)
                            umma_f16(tacc + S::UN, umma_smem_desc(a_addr + GM_STAGE_A + k * 32),
                                     umma_smem_desc(b_addr + k * 32), idesc, kb > kb0 || k > 0);
                    }
                    umma_commit(&a_empty[s]);
                    umma_commit(&b_empty[b]);
                }
                if (!ok) break;
                umma_commit(&acc_full[as]);
                ++ti;
            }
        }
    } else if (warp < GQ_FIRST_EXPAND) {
        gemm_epilogue_loop<EPI, S::UN, S::ACC, 2>(a, tmem, acc_full, acc_empty, warp, lane, total, epi_scratch, tab);
    } else {
        // eight expanding warps: thread -> (B row, which 32 of the block's 64 weights)
        const int x = threadIdx.x - GQ_FIRST_EXPAND * 32, row_t = x & 127, hh = x >> 7;
        uint32_t it = 0, sbi = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
            GemmTile w;
            if (!gemm_tile_at(a, tab, t, w)) continue;
            const int kb0 = w.split * a.kb_split, kb1 = min(KB_ALL, kb0 + a.kb_split);
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const int j = kb & 3, b = it % S::SB;
                if (j == 0) ++sbi;                    // sbi - 1 is the super-block in use
                const int p = (sbi - 1) % S::SP;
                if (j == 0) ok = mbar_wait(&p_full[p], ((sbi - 1) / S::SP) & 1, a.status);
                if (ok && it >= S::SB) ok = mbar_wait(&b_empty[b], ((it / S::SB) - 1) & 1, a.status);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint8_t* packed = sm_p + (size_t)p * S::PACKED;
                uint8_t* tile = sm_b + (size_t)b * S::B16;
#pragma unroll
                for (int rr = 0; rr < S::UN / 128; ++rr) {
                    const int r = row_t + rr * 128;
                    dequant_half_block<KIND>(packed + (size_t)r * S::SBB, j, hh, tile, r);
                }
                fence_proxy_async();                  // generic-proxy stores -> visible to the MMA
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&b_full[b]);
                    if (j == 3) mbar_arrive(&p_empty[p]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, S::ACC * 2 * S::UN);
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

// A producer that has already written a block of fp32 rows once more as fp16 (a fused norm)
// registers the copy; the next un-gathered pack of exactly that block is then skipped and the
// GEMM reads the copy.  One entry, owned by the thread that drives the library; the producer's
// caller clears it as soon as the rows' consumers have been enqueued.
static struct { const float* src; const __half* rows16; int64_t rows; int K; } g_f16_shadow = {nullptr, nullptr, 0, 0};
void f16_shadow_set(const float* src, const __half* rows16, int64_t rows, int K) { g_f16_shadow = {src, rows16, rows, K}; }
void f16_shadow_clear() { g_f16_shadow = {nullptr, nullptr, 0, 0}; }
const __half* f16_shadow_find(const float* src, int64_t rows, int K) {
    return (src && g_f16_shadow.src == src && g_f16_shadow.rows == rows && g_f16_shadow.K == K) ? g_f16_shadow.rows16 : nullptr;
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

// Tensor map over packed rows viewed as 32-bit words: boxes of (box_bytes / 4) words
// x GM_TILE_N rows, no swizzle.
static int make_packed_map(CUtensorMap* out, const void* base, int64_t rows, int64_t row_bytes, int box_bytes) {
    B200_REQUIRE(base && rows > 0 && row_bytes % 16 == 0 && box_bytes % 16 == 0, "packed map: rows must be 16-byte multiples");
    B200_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "packed map: base must be 16-byte aligned");
    typedef std::tuple<const void*, int64_t, int64_t, int> Key;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const Key key(base, rows, row_bytes, box_bytes);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return B200_OK;
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(B200_ECUDA, "packed map: the driver does not export cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 4), (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)(box_bytes / 4), (cuuint32_t)GM_TILE_N};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200_ECUDA, "packed map: cuTensorMapEncodeTiled failed with %d", (int)r);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return B200_OK;
}

// c[m, n] = sum over the splits, in split order (deterministic), of the partial products.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, float* __restrict__ c, int splits,
                                                           int64_t stride, int M, int N, int64_t ldc) {
    const int64_t total = (int64_t)M * N;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / N, o = m * ldc + (i - m * N);
        float v = part[o];
        for (int s = 1; s < splits; ++s) v += part[s * stride + o];
        c[o] = v;
    }
}

template <int EPI, int KIND>
static int launch_gemm_q(const GemmArgs& a) {
    using S = GemmQShape<EPI, KIND>;
    auto kern = umma_gemm_q_kernel<EPI, KIND>;
    static bool configured = false;
    if (!configured) {
        B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM));
        configured = true;
    }
    GemmArgs b = a;
    b.tile_m = 2 * GM_TILE_M;
    b.m_slots = (a.M + b.tile_m - 1) / b.tile_m + (a.offsets ? a.groups : 0);
    b.tile_n = GemmShape<EPI>::TN;
    b.n_tiles = (a.N + b.tile_n - 1) / b.tile_n;
    b.k_splits = 1;
    b.kb_split = a.K / GM_TILE_K;
    b.split_stride = 0;
    // Few tiles (few rows and a narrow matrix: batched decode, the attention projections):
    // every CTA would stream its 128 weight rows over all of K while most SMs idle, so K is
    // cut across CTAs and the partial products are added afterwards in a fixed order.
    const int tiles = b.m_slots * b.n_tiles, sb = a.K / 256;
    // Not for the grouped form: the reduction pass walks all M rows, but a grouped launch
    // writes partial sums only for the rows its offsets cover - rows outside them (other
    // ranks' experts in the expert-parallel layer) must be left exactly as they are.
    if (EPI == GEMM_EPI_STORE && a.offsets == nullptr && a.allow_split_k && sb >= 2 && tiles * 2 <= num_sms()) {
        const int want = std::min(sb, num_sms() / tiles);
        const int per = (sb + want - 1) / want;
        b.k_splits = (sb + per - 1) / per;
        b.kb_split = per * 4;
    }
    if (b.k_splits > 1) {
        b.split_stride = (int64_t)a.M * a.ldc;
        void* wsp;
        int rc = workspace(WS_SPLITK).ensure((size_t)b.k_splits * b.split_stride * sizeof(float) + 256, &wsp);
        if (rc) return rc;
        b.c = static_cast<float*>(wsp);
    }
    const int grid = std::min(tiles * b.k_splits, num_sms());
    kern<<<grid, GQ_THREADS, S::SMEM, stream()>>>(b);
    B200_LAUNCH_CHECK("umma_gemm_q_kernel");
    if (b.k_splits > 1) {
        const int64_t total = (int64_t)a.M * a.N;
        splitk_reduce_kernel<<<(unsigned)std::min<int64_t>(ceil_div64(total, 256), (int64_t)num_sms() * 8), 256, 0, stream()>>>(
            b.c, a.c, b.k_splits, b.split_stride, a.M, a.N, a.ldc);
        B200_LAUNCH_CHECK("splitk_reduce_kernel");
    }
    return B200_OK;
}

// As umma_gemm(), with B (and B2) packed in `kind` (0..3), [b_rows, K]; K % 256 == 0.
int umma_gemm_q(int epi, int kind, const __half* A, int64_t a_rows, const void* B, const void* B2, int64_t b_rows,
                const int32_t* offsets, int groups, int M, int N, int K, float* c, __half* c16, int64_t ldc,
                float scale, const int32_t* group_map, float* const* group_c, bool allow_split_k) {
    if (M <= 0 || N <= 0) return B200_OK;
    B200_REQUIRE(kind >= 0 && kind <= 3, "umma_gemm_q: unknown kind %d", kind);
    B200_REQUIRE(!group_c || (offsets && epi == GEMM_EPI_STORE), "umma_gemm_q: per-group outputs need the grouped store form");
    B200_REQUIRE(A && B && K > 0 && K % 256 == 0, "umma_gemm_q: K must be a positive multiple of 256");
    B200_REQUIRE(groups >= 1 && (offsets || groups == 1), "umma_gemm_q: groups need a device offsets array");
    B200_REQUIRE((group_map || b_rows >= (int64_t)groups * N) && a_rows >= M, "umma_gemm_q: operand shapes do not cover the groups");
    GemmArgs a;
    int rc = make_tile_map(&a.map_a, A, a_rows, K, GM_TILE_M);
    if (rc) return rc;
    const int64_t row_bytes = q_row_bytes(kind, K);
    const int sbb = 8 * (kind == 3 ? 18 : q_block_bytes(kind));
    rc = make_packed_map(&a.map_b, B, b_rows, row_bytes, sbb);
    if (rc) return rc;
    a.map_b2 = a.map_b;
    if (epi == GEMM_EPI_SWIGLU) {
        B200_REQUIRE(B2 && c16 && ldc % 2 == 0, "umma_gemm_q: the SwiGLU form needs the second matrix and an fp16 output");
        rc = make_packed_map(&a.map_b2, B2, b_rows, row_bytes, sbb);
        if (rc) return rc;
    } else {
        B200_REQUIRE(c || group_c, "umma_gemm_q: null output");
    }
    a.offsets = offsets; a.group_map = group_map; a.M = M; a.groups = groups; a.N = N; a.K = K;
    a.c = c; a.c16 = c16; a.ldc = ldc; a.scale = scale; a.group_c = group_c; a.allow_split_k = allow_split_k;
    a.status = stream_status_ptr();
    B200_REQUIRE(a.status, "umma_gemm_q: status word allocation failed");
    // wide store tiles when they still fill the machine (row slots are an upper bound when
    // grouped) and K is long: this kernel's wide form has a single accumulator set, so its
    // epilogue is not hidden, which costs more than the wide MMA gains when a tile has only a
    // few K steps (measured: the K = 512 expert down-projections lose 20 %, K = 1536 gains 16 %)
    const int slots256 = (M + 2 * GM_TILE_M - 1) / (2 * GM_TILE_M) + (offsets ? groups / 2 : 0);
    const bool wide = epi == GEMM_EPI_STORE && N >= 2 * GM_TILE_N && K >= 1024 &&
                      slots256 * ((N + 2 * GM_TILE_N - 1) / (2 * GM_TILE_N)) >= num_sms();
#define GQ(KIND_)                                                                        \
    return epi == GEMM_EPI_SWIGLU ? launch_gemm_q<GEMM_EPI_SWIGLU, KIND_>(a)             \
           : wide                 ? launch_gemm_q<GEMM_EPI_STORE_WIDE, KIND_>(a)         \
                                  : launch_gemm_q<GEMM_EPI_STORE, KIND_>(a);
    switch (kind) {
        case 0: GQ(0)
        case 1: GQ(1)
        case 2: GQ(2)
        default: GQ(3)
    }
#undef GQ
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
    GemmArgs b = a;
    b.tile_m = GM_TILE_M;
    b.m_slots = (a.M + b.tile_m - 1) / b.tile_m + (a.offsets ? a.groups : 0);
    b.tile_n = GemmShape<EPI>::TN;
    b.n_tiles = (a.N + b.tile_n - 1) / b.tile_n;
    b.k_splits = 1;
    b.kb_split = 0;
    b.split_stride = 0;
    const int grid = std::min(b.m_slots * b.n_tiles, num_sms());
    kern<<<grid, GM_THREADS, S::SMEM, stream()>>>(b);
    B200_LAUNCH_CHECK("umma_gemm_kernel");
    return B200_OK;
}

// A [a_rows, K] fp16; B (and B2) [b_rows, K] fp16 with b_rows = groups * N.
// offsets: device [groups + 1] or null (then groups must be 1 and all M rows form it).
int umma_gemm(int epi, const __half* A, int64_t a_rows, const __half* B, const __half* B2, int64_t b_rows,
              const int32_t* offsets, int groups, int M, int N, int K, float* c, __half* c16, int64_t ldc, float scale,
              const int32_t* group_map, float* const* group_c) {
    if (M <= 0 || N <= 0) return B200_OK;
    B200_REQUIRE(A && B && K > 0 && K % 8 == 0, "umma_gemm: K must be a positive multiple of 8");
    B200_REQUIRE(!group_c || (offsets && epi == GEMM_EPI_STORE), "umma_gemm: per-group outputs need the grouped store form");
    B200_REQUIRE(groups >= 1 && (offsets || groups == 1), "umma_gemm: groups need a device offsets array");
    B200_REQUIRE((group_map || b_rows >= (int64_t)groups * N) && a_rows >= M, "umma_gemm: operand shapes do not cover the groups");
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
        B200_REQUIRE(c || group_c, "umma_gemm: null output");
    }
    a.offsets = offsets; a.group_map = group_map; a.M = M; a.groups = groups; a.N = N; a.K = K;
    a.c = c; a.c16 = c16; a.ldc = ldc; a.scale = scale; a.group_c = group_c; a.allow_split_k = false;
    a.status = stream_status_ptr();
    B200_REQUIRE(a.status, "umma_gemm: status word allocation failed");
    const int slots128 = (M + GM_TILE_M - 1) / GM_TILE_M + (offsets ? groups / 2 : 0);
    const bool wide = epi == GEMM_EPI_STORE && N >= 2 * GM_TILE_N && slots128 * ((N + 2 * GM_TILE_N - 1) / (2 * GM_TILE_N)) >= num_sms();
    return epi == GEMM_EPI_SWIGLU ? launch_gemm<GEMM_EPI_SWIGLU>(a)
           : wide                 ? launch_gemm<GEMM_EPI_STORE_WIDE>(a)
                                  : launch_gemm<GEMM_EPI_STORE>(a);
}

}  // namespace b200
