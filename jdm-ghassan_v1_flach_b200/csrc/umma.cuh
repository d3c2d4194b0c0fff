// Inline-PTX wrappers for the Blackwell tensor-core path: tcgen05 (MMA issued by one
// thread, accumulators in tensor memory), 2-D TMA tile loads with the 128-byte
// swizzle the MMA's shared-memory descriptors expect, and the descriptor encodings.
//
// Operand tiles are "K-major": a row of the tile holds 64 consecutive fp16 values of
// K (128 bytes).  Eight rows form a 1024-byte swizzle atom in which the 16-byte
// chunk c of row r is stored at chunk position c ^ (r & 7); atoms are stacked along
// the row dimension 1024 bytes apart.  A 2-D TMA load with SWIZZLE_128B produces
// exactly this, and so does swz128_offset() for tiles written by threads.
#pragma once

#include <cuda.h>

#include "stream.cuh"

namespace b200 {

// Byte offset of element (row, k) (k in halves, 0..63) inside a K-major SW128 tile.
__host__ __device__ inline uint32_t swz128_offset(int row, int k) {
    const int chunk = (k >> 3) ^ (row & 7);
    return (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u + (uint32_t)chunk * 16u + (uint32_t)(k & 7) * 2u;
}

// Instruction descriptor of tcgen05.mma.kind::f16 with fp16 A and B (both K-major)
// and fp32 accumulation: c_format [4,6) = 1, a_format [7,10) = 0, b_format [10,13) = 0,
// a_major bit 15 = 0, b_major bit 16 = 0, N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_f16(int M, int N) {
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

#ifdef __CUDACC__
// Shared-memory matrix descriptor of a K-major SW128 tile starting at `smem_addr`
// (1024-byte aligned, plus a multiple of 32 bytes to step along K inside the atom):
// start address >> 4 in [0,14), leading byte offset (unused for swizzled K-major) = 1
// in [16,30), stride byte offset = 1024 >> 4 in [32,46), version 1 in [46,48),
// layout type SWIZZLE_128B = 2 in [61,64).
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, one thread issues.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// The mbarrier receives one arrival when every MMA issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 32 consecutive fp32 columns of this warp's 32 accumulator rows (lane = row).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// 2-D tile load (no multicast).  x = element coordinate along K (a multiple of 8 so
// the copy starts on a 16-byte boundary), y = row.  Out-of-range parts read as zero.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// Makes shared-memory writes of this thread visible to the async proxy (TMA, tcgen05).
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
#endif

// Host: tensor map of a row-major fp16 matrix [rows, K] with boxes of 64 x box_rows
// and the 128-byte swizzle.  Returns B200_OK or an error status.
int make_tile_map(CUtensorMap* out, const void* base, int64_t rows, int64_t K, int box_rows);

}  // namespace b200
