// tcgen05 (5th-gen tensor core) + TMEM primitives for sm_100a, as thin inline-PTX wrappers.
//
// Shared-memory operands use the un-swizzled canonical ("interleaved") layout, which is convenient
// when the operands are produced by CUDA cores rather than by TMA: a *core matrix* is 8 rows x 16
// bytes stored as 128 contiguous bytes;
//   K-major  operand: core (rb, kb) covers rows 8rb..8rb+7 and K-bytes 16kb..16kb+15; inside it row r
//                     sits at +16r.
//   MN-major operand: core (mb, kb) covers MN-elements [T*mb, T*mb+T) (T = 16 / element size) and
//                     K-rows 8kb..8kb+7; inside it K-row r sits at +16r, MN-elements are contiguous.
// In both cases the descriptor's SBO is the byte distance between cores adjacent along M/N and LBO the
// byte distance between cores adjacent along K. One MMA instruction consumes 32 bytes of K (K-major)
// or two cores of 8 K-rows for 16-bit types / one core for tf32 (MN-major).
#pragma once
#include <stdint.h>

namespace kda {
namespace umma {

constexpr uint32_t FMT_F16 = 0, FMT_BF16 = 1, FMT_TF32 = 2;

// 32-bit instruction descriptor: fp32 accumulate, dense, no negate.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt_ab, int M, int N, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (fmt_ab << 7) | (fmt_ab << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// 64-bit shared-memory matrix descriptor, no swizzle.
__device__ __forceinline__ uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
           (1ull << 46);
}

// ---- TMEM allocation: executed by ONE full warp; the base address lands in shared memory ----
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; issued by a single thread.
__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                 :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Make the mbarrier track completion of all MMAs this thread issued so far (one arrival).
__device__ __forceinline__ void commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"((uint32_t)__cvta_generic_to_shared(bar)) : "memory");
}

// TMEM -> registers: warp w of a warpgroup reads lanes 32(w%4).. ; thread i gets lane 32(w%4)+i,
// 16 consecutive 32-bit columns starting at the address's column.
__device__ __forceinline__ void ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace umma
}  // namespace kda
