// MoE layer for a decode batch (tens of tokens): the experts as weight streams shared by
// the tokens that chose them.
//
// With 64 tokens and top-6 of 64 experts nearly every expert is touched, by about six tokens
// each.  The tensor-core GEMM path would expand a 128-row weight tile per expert for six
// rows of activations; the token-major few-token path (fused_moe.cu) would stream an expert
// once per token.  Here the (token, k) slots are sorted by expert (the layer's own
// permutation), cut into *units* of up to eight slots of one expert, and a unit is served
// by a few CTAs that stage its tokens' activations once and stream the expert's rows
// through the few-token dot engine (mma.sync on exact nibbles, eight token columns): every
// expert's bytes cross HBM once, the arithmetic is the few-token path's (exact dequantised
// weights, activations as fp16 head + tail pairs, fp32 accumulation).
//
//   moe_units_build_kernel    offsets -> unit table (expert, first sorted slot, slots)
//   moe_units_gateup_kernel   act[slot, :] = silu(gate_e x_t) * up_e x_t          [NK, E]
//   moe_units_down_kernel     y[slot, :]   = down_e act[slot, :]                  [NK, d]
// The weighted combination over a token's K slots (k order) and the shared expert are the
// many-token path's (moe_grouped.cu).  Arithmetic followed: core/moe_cpu.cpp:198-288.
#include "fused_common.cuh"
#include "gemm.cuh"

namespace b200 {

constexpr int UNIT_SLOTS = 8;        // token columns of the dot engine
// Rows carved for a unit's activations.  Tensor-core kinds: the columns of absent tokens are never
// read back, so they may multiply any staged row - token 0 stands in and no zero row is kept
// (xact_carve adds one row to its count: UNIT_SLOTS rows in all), which leaves room for a third
// ring stage next to eight tokens.
template <int KIND>
struct UnitRows {
    static constexpr int value = UsesMma<KIND>::value ? UNIT_SLOTS - 1 : UNIT_SLOTS;
};

struct MoeUnitArgs {
    const float* x = nullptr;            // [T, d] layer input
    const int32_t* grouped = nullptr;    // [NK] slot numbers sorted by expert (slot / K = token)
    const int4* units = nullptr;         // (expert, first sorted position, slots <= 8, -)
    const int* n_units = nullptr;
    const uint8_t *gates = nullptr, *ups = nullptr, *downs = nullptr;
    float* act = nullptr;                // [NK, E], sorted order
    float* y = nullptr;                  // [NK, d], sorted order
    int d = 0, E = 0, K = 0;
    int rows_per_tile = 0, stage_bytes = 0, n_stages = 0;
    int row_tiles = 1;                   // down kernel, tensor-core kinds: 16-row tiles per ring entry
    int* status = nullptr;
    bool dry = false;
};

// One block; ne <= 256 experts.
__global__ void moe_units_build_kernel(const int32_t* __restrict__ offsets, int ne, int4* __restrict__ units,
                                       int* __restrict__ n_units) {
    __shared__ int first[257];
    const int e = threadIdx.x;
    int chunks = 0;
    if (e < ne) chunks = (offsets[e + 1] - offsets[e] + UNIT_SLOTS - 1) / UNIT_SLOTS;
    first[e + 1] = chunks;
    __syncthreads();
    if (threadIdx.x == 0) {
        first[0] = 0;
        for (int i = 1; i <= ne; ++i) first[i] += first[i - 1];
        *n_units = first[ne];
    }
    __syncthreads();
    if (e < ne) {
        const int lo = offsets[e], hi = offsets[e + 1];
        for (int c = 0; c < chunks; ++c) {
            const int p0 = lo + c * UNIT_SLOTS;
            units[first[e] + c] = make_int4(e, p0, min(UNIT_SLOTS, hi - p0), 0);
        }
    }
}

// grid (ctas per unit, unit slots).  An output tile is R rows of the activation; its two weight
// tiles - R rows of the expert's gate matrix, the same R rows of its up matrix - travel as two
// consecutive ring entries (2 i, 2 i + 1), which keeps a stage small enough that two CTAs fit
// an SM next to eight tokens' staged activations.
template <int KIND>
__global__ void __launch_bounds__(SG_THREADS, 2) moe_units_gateup_kernel(MoeUnitArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    Ring ring;
    ring.stages = smem;
    ring.stage_bytes = a.stage_bytes;
    ring.n_stages = a.n_stages;
    ring.status = a.status;
    XAct xa;
    uint8_t* p = xact_carve<KIND>(xa, smem + (size_t)a.n_stages * a.stage_bytes, a.d, UnitRows<KIND>::value, false);
    xa.zrow = 0;
    float* red = reinterpret_cast<float*>(p);
    p += (size_t)RED_FLOATS * 4;
    ring.full = reinterpret_cast<uint64_t*>(p);
    ring.empty = ring.full + SG_MAX_STAGES;
    double* red_d = reinterpret_cast<double*>(ring.empty + SG_MAX_STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    ring.init();
    if (threadIdx.x == 0) pdl_launch_dependents();
    pdl_wait();                                   // the unit table comes from the kernels before
    if ((int)blockIdx.y >= *a.n_units) return;
    const int4 unit = a.units[blockIdx.y];
    const int e = unit.x, p0 = unit.y, M = unit.z;
    const int num_tiles = (a.E + a.rows_per_tile - 1) / a.rows_per_tile;
    const int first = blockIdx.x, step = gridDim.x;
    const int n_my = first < num_tiles ? (num_tiles - first + step - 1) / step : 0;
    const int64_t rb = row_bytes_of(KIND, a.d);

    if (warp == SG_CONSUMERS) {
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < 2 * n_my; ++i) {
                if (!ring.acquire(i)) break;
                const int r0 = (first + (i >> 1) * step) * a.rows_per_tile;
                const int rows = min(a.rows_per_tile, a.E - r0);
                const int64_t row0 = (int64_t)e * a.E + r0;
                const uint32_t bytes = (uint32_t)(rows * rb);
                ring.expect(i, bytes);
                ring.copy(i, 0, ((i & 1) ? a.ups : a.gates) + row0 * rb, bytes);
                issued = i + 1;
            }
            ring.drain(issued);
        }
        return;
    }
    // the unit's tokens in one pass: every load in flight before the first is used, one barrier
    stage_rows<KIND, false, SG_CONSUMERS, 12>(a.x, a.d, xa, M, red_d, a.grouped + p0, a.K);
    const int e_row = threadIdx.x >> 3, e_m = threadIdx.x & 7;
    for (int i = 0; i < n_my; ++i) {
        const int r0 = (first + i * step) * a.rows_per_tile;
        const int rows = min(a.rows_per_tile, a.E - r0);
        float* red_buf = red + (size_t)(i & 1) * RED_BUF;
        if (!ring.wait_full(2 * i)) break;
        tile_compute<KIND, UNIT_SLOTS>(ring.stage(2 * i), rb, rows, a.d, xa, 0, M, red_buf, warp, lane);
        ring.release(2 * i);
        if (!ring.wait_full(2 * i + 1)) break;
        tile_compute<KIND, UNIT_SLOTS>(ring.stage(2 * i + 1), rb, rows, a.d, xa, 0, M, red_buf + RED_PASS, warp, lane);
        ring.release(2 * i + 1);
        consumer_sync();
        if (e_row < rows && e_m < M) {
            const float g = red_value<KIND>(red_buf, e_row, e_m);
            const float u = red_value<KIND>(red_buf + RED_PASS, e_row, e_m);
            a.act[(int64_t)(p0 + e_m) * a.E + r0 + e_row] = silu_acc(g) * u;
        }
    }
}

// grid (ctas per unit, unit slots).  A tile: R rows of the expert's down matrix (K = E).
template <int KIND>
__global__ void __launch_bounds__(SG_THREADS, 2) moe_units_down_kernel(MoeUnitArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    Ring ring;
    ring.stages = smem;
    ring.stage_bytes = a.stage_bytes;
    ring.n_stages = a.n_stages;
    ring.status = a.status;
    XAct xa;
    uint8_t* p = xact_carve<KIND>(xa, smem + (size_t)a.n_stages * a.stage_bytes, a.E, UnitRows<KIND>::value, false);
    xa.zrow = 0;
    float* red = reinterpret_cast<float*>(p);
    p += (size_t)RED_FLOATS * 4;
    ring.full = reinterpret_cast<uint64_t*>(p);
    ring.empty = ring.full + SG_MAX_STAGES;
    double* red_d = reinterpret_cast<double*>(ring.empty + SG_MAX_STAGES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    ring.init();
    if (threadIdx.x == 0) pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.y >= *a.n_units) return;
    const int4 unit = a.units[blockIdx.y];
    const int e = unit.x, p0 = unit.y, M = unit.z;
    const int num_tiles = (a.d + a.rows_per_tile - 1) / a.rows_per_tile;
    const int first = blockIdx.x, step = gridDim.x;
    const int n_my = first < num_tiles ? (num_tiles - first + step - 1) / step : 0;
    const int64_t rb = row_bytes_of(KIND, a.E);

    if (warp == SG_CONSUMERS) {
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < n_my; ++i) {
                if (!ring.acquire(i)) break;
                const int r0 = (first + i * step) * a.rows_per_tile;
                const int rows = min(a.rows_per_tile, a.d - r0);
                const uint32_t bytes = (uint32_t)(rows * rb);
                ring.expect(i, bytes);
                ring.copy(i, 0, a.downs + ((int64_t)e * a.d + r0) * rb, bytes);
                issued = i + 1;
            }
            ring.drain(issued);
        }
        return;
    }
    stage_rows<KIND>(a.act + (int64_t)p0 * a.E, a.E, xa, M, red_d);
    const int e_row = threadIdx.x >> 3, e_m = threadIdx.x & 7;
    if constexpr (UsesMma<KIND>::value) {
        // A ring entry holds RT 16-row tiles; warp = (tile rt, K part kp of KP = 8 / RT), so a warp
        // runs RT times the groups of a one-tile entry between two hand-overs and the parts to add
        // afterwards are KP, not eight.  red: [kp][rt][16 rows][8 tokens].
        const int RT = a.row_tiles, KP = SG_CONSUMERS / RT;
        const int rt = warp / KP, kp = warp - rt * KP;
        const XHalf xh = xa.half();
        for (int i = 0; i < n_my; ++i) {
            if (!ring.wait_full(i)) break;
            const int r0 = (first + i * step) * a.rows_per_tile;
            const int rows = min(a.rows_per_tile, a.d - r0);
            float* red_buf = red + (size_t)(i & 1) * RED_BUF;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const uint8_t* sub = ring.stage(i) + (size_t)rt * TILE_ROWS * rb;
            if (rt * TILE_ROWS < rows) {
                if (KIND == 3) tile_dot_q4k(sub, (int)rb, a.E, xh, M, kp, KP, lane, acc);
                else tile_dot_f16(sub, (int)rb, a.E, xh, M, kp, KP, lane, acc);
            }
            float* o = red_buf + (size_t)(kp * RT + rt) * RED_PASS;
            const int gid = lane >> 2, c = 2 * (lane & 3);
            o[gid * RED_TOK + c] = acc[0];
            o[gid * RED_TOK + c + 1] = acc[1];
            o[(gid + 8) * RED_TOK + c] = acc[2];
            o[(gid + 8) * RED_TOK + c + 1] = acc[3];
            ring.release(i);
            consumer_sync();
            for (int row = e_row; row < rows; row += SG_CTHREADS / RED_TOK) {
                if (e_m < M) {
                    const float* src = red_buf + (size_t)(row >> 4) * RED_PASS + (row & 15) * RED_TOK + e_m;
                    float v = 0.0f;
                    for (int q = 0; q < KP; ++q) v += src[(size_t)q * RT * RED_PASS];
                    a.y[(int64_t)(p0 + e_m) * a.d + r0 + row] = v;
                }
            }
        }
    } else {
        for (int i = 0; i < n_my; ++i) {
            if (!ring.wait_full(i)) break;
            const int r0 = (first + i * step) * a.rows_per_tile;
            const int rows = min(a.rows_per_tile, a.d - r0);
            float* red_buf = red + (size_t)(i & 1) * RED_BUF;
            tile_compute<KIND, UNIT_SLOTS>(ring.stage(i), rb, rows, a.E, xa, 0, M, red_buf, warp, lane);
            ring.release(i);
            consumer_sync();
            if (e_row < rows && e_m < M) a.y[(int64_t)(p0 + e_m) * a.d + r0 + e_row] = red_value<KIND>(red_buf, e_row, e_m);
        }
    }
}

template <int KIND>
static int moe_units_kind(MoeUnitArgs a, int max_units) {
    const int64_t rb_d = row_bytes_of(KIND, a.d), rb_e = row_bytes_of(KIND, a.E);
    const size_t fixed = (size_t)RED_FLOATS * 4 + BAR_BYTES + 64;
    // enough CTAs per unit that the launch covers the machine about three times over
    const int per_unit = std::max(1, std::min(8, (3 * num_sms() + max_units - 1) / max_units));
    int rc;
    {
        MoeUnitArgs g = a;
        const int R = pick_rows(KIND, rb_d, rb_d, rb_d, a.E);
        if (R < 1 || !tail_tile_ok(a.E, R, rb_d)) return fail(B200_EUNSUPPORTED, "moe_units: row size cannot be tiled to 16 bytes");
        g.rows_per_tile = R;
        g.stage_bytes = (int)(((size_t)R * rb_d + 127) / 128 * 128);
        const size_t other = xact_bytes<KIND>(a.d, UnitRows<KIND>::value, false) + fixed;
        // two resident CTAs per SM matter more here than a deep ring (the tiles of a unit are
        // consecutive rows: the stream has no gaps to hide): two stages in half an SM's shared
        // memory are taken before more stages in all of it
        g.n_stages = pick_stages_in(g.stage_bytes, other, SMEM_BUDGET);
        if (g.n_stages < 2) g.n_stages = pick_stages_in(g.stage_bytes, other, SMEM_BUDGET_FULL);
        if (g.n_stages < 2) return fail(B200_EUNSUPPORTED, "moe_units: hidden size %d does not fit the shared-memory staging", a.d);
        auto kern = moe_units_gateup_kernel<KIND>;
        static bool cfgd = false;
        if (!cfgd) { rc = allow_smem(kern); if (rc) return rc; cfgd = true; }
        const int gx = std::min(per_unit, ceil_div(a.E, R));
        rc = launch_pdl(kern, dim3(gx, max_units), dim3(SG_THREADS), (size_t)g.n_stages * g.stage_bytes + other, g);
        if (rc) return rc;
    }
    {
        MoeUnitArgs g = a;
        int R = pick_rows(KIND, rb_e, rb_e, rb_e, a.d);
        if (UsesMma<KIND>::value) {
            // short contractions: several 16-row tiles per ring entry, so that a warp has about four
            // groups of 64 to run per entry (E = 512: four tiles, two K parts)
            const int groups = std::max(1, a.E / 64);
            g.row_tiles = groups <= 8 ? 4 : groups <= 16 ? 2 : 1;
            while (g.row_tiles > 1 && (a.d < R * g.row_tiles || !tail_tile_ok(a.d, R * g.row_tiles, rb_e))) g.row_tiles /= 2;
            R *= g.row_tiles;
        }
        if (R < 1 || !tail_tile_ok(a.d, R, rb_e)) return fail(B200_EUNSUPPORTED, "moe_units: row size cannot be tiled to 16 bytes");
        g.rows_per_tile = R;
        g.stage_bytes = (int)(((size_t)R * rb_e + 127) / 128 * 128);
        const size_t other = xact_bytes<KIND>(a.E, UnitRows<KIND>::value, false) + fixed;
        g.n_stages = pick_stages(g.stage_bytes, other);
        if (g.n_stages < 2) return fail(B200_EUNSUPPORTED, "moe_units: expert width %d does not fit the shared-memory staging", a.E);
        auto kern = moe_units_down_kernel<KIND>;
        static bool cfgd = false;
        if (!cfgd) { rc = allow_smem(kern); if (rc) return rc; cfgd = true; }
        const int gx = std::min(per_unit, ceil_div(a.d, R));
        rc = launch_pdl(kern, dim3(gx, max_units), dim3(SG_THREADS), (size_t)g.n_stages * g.stage_bytes + other, g);
        if (rc) return rc;
    }
    return B200_OK;
}

// The routed experts of N tokens whose slots have been sorted by expert: grouped / offsets as
// moe_dispatch_perm leaves them; act [N K, E] and y [N K, d] fp32 in sorted order; units:
// scratch for unit_table_bytes(N K, ne) bytes.  kind: a packed kind or KIND_F16.
size_t moe_units_table_bytes(int64_t NK, int ne) { return ((size_t)(ne + NK / UNIT_SLOTS + 1) * sizeof(int4) + 255) / 256 * 256 + 256; }
int moe_units_forward(const float* x, const int32_t* grouped, const int32_t* offsets, const void* gates, const void* ups,
                      const void* downs, float* act, float* y, void* units_scratch, int64_t N, int d, int E, int ne, int K,
                      int kind) {
    B200_REQUIRE(ne <= 256 && N * K <= 0x7fffffff, "moe_units: too many experts or slots");
    B200_REQUIRE(d % 32 == 0 && E % 32 == 0, "moe_units: d and E must be multiples of 32");
    if (kind == 3) B200_REQUIRE(d % 256 == 0 && E % 256 == 0, "moe_units: Q4_K needs multiples of 256");
    const int max_units = (int)(ne + (N * K) / UNIT_SLOTS);
    B200_REQUIRE(max_units <= 65535, "moe_units: too many units");
    int* n_units = static_cast<int*>(units_scratch);
    int4* units = reinterpret_cast<int4*>(static_cast<char*>(units_scratch) + 256);
    moe_units_build_kernel<<<1, 256, 0, stream()>>>(offsets, ne, units, n_units);
    B200_LAUNCH_CHECK("moe_units_build_kernel");
    MoeUnitArgs a;
    a.x = x; a.grouped = grouped; a.units = units; a.n_units = n_units;
    a.gates = static_cast<const uint8_t*>(gates); a.ups = static_cast<const uint8_t*>(ups);
    a.downs = static_cast<const uint8_t*>(downs);
    a.act = act; a.y = y; a.d = d; a.E = E; a.K = K;
    a.status = stream_status_ptr();
    B200_REQUIRE(a.status, "moe_units: status word allocation failed");
    switch (kind) {
        case 0: return moe_units_kind<0>(a, max_units);
        case 1: return moe_units_kind<1>(a, max_units);
        case 2: return moe_units_kind<2>(a, max_units);
        case 3: return moe_units_kind<3>(a, max_units);
        case KIND_F16: return moe_units_kind<KIND_F16>(a, max_units);
        default: return fail(B200_EUNSUPPORTED, "moe_units: fp32 experts take the token-major path");
    }
}

}  // namespace b200
