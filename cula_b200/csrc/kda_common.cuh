// Shared definitions for the sm_100a KDA kernels: tile-pack layout, swizzles, PTX wrappers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kda {

constexpr int BT = 64;    // chunk length (tokens); fixed at 64 as in cula/kda/chunk.py:54
constexpr int DK = 128;   // key head dim
constexpr int DV = 128;   // value head dim
constexpr float RCP_LN2 = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------------------------
// Forward tile pack: everything the state scan needs for one (chunk, head), contiguous in HBM so
// that one stage of the scan pipeline is two bulk copies. Each array is stored in the exact image
// the scan wants in shared memory: row-major with the 16-byte column groups XOR-swizzled by
// (row & 7), which makes every ldmatrix read bank-conflict free.
//   W    [64][128] fp16   w  = Akk (beta k 2^g)
//   QG   [64][128] fp16   qg = scale * q 2^g
//   KG   [64][128] fp16   kg = k 2^(g_last - g)
//   AQK  [64][64]  fp16   scale * tril(q k^T gated)
//   DECAY[128]     fp32   2^(g_last)
//   U0,U1 [64][64] fp16   u = Akk (beta v), value columns 0..63 and 64..127
// ---------------------------------------------------------------------------------------------
constexpr int TP_W = 0;
constexpr int TP_QG = 16384;
constexpr int TP_KG = 32768;
constexpr int TP_AQK = 49152;
constexpr int TP_DECAY = 57344;
constexpr int TP_U0 = 57856;
constexpr int TP_U1 = 66048;
constexpr int TP_BYTES = 74240;
constexpr int TP_HEAD_BYTES = TP_U0;   // W..DECAY: shared by both value halves

// byte offset of element (row, col) of a 2-byte matrix with 128 columns (256-byte rows)
__host__ __device__ __forceinline__ int swz256(int row, int col) {
    return row * 256 + ((((col >> 3) ^ (row & 7))) << 4) + ((col & 7) << 1);
}
// same for 64 columns (128-byte rows)
__host__ __device__ __forceinline__ int swz128(int row, int col) {
    return row * 128 + ((((col >> 3) ^ (row & 7))) << 4) + ((col & 7) << 1);
}

// Status word values written by kernels whose bounded waits give up.
constexpr int STATUS_OK = 0;
constexpr int STATUS_WAIT_TIMEOUT = 1;
constexpr int STATUS_BAD_INDEX = 2;        // a state-pool index past the end of the pool (decode)
constexpr int STATUS_RANGE = 3;            // a forward intermediate left the fp16 range (or is not finite)

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" :: "l"(p));
}
// one instruction asks for a whole contiguous range (16-byte aligned, a multiple of 16 bytes) to be brought into L2
__device__ __forceinline__ void bulk_prefetch_l2(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(p), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// true if either fp16 half of x is +-inf or NaN (exponent bits all ones)
__device__ __forceinline__ bool f16x2_not_finite(uint32_t x) {
    return __vcmpeq2(x & 0x7c007c00u, 0x7c007c00u) != 0u;
}
__device__ __forceinline__ float2 unpack_f16(uint32_t x) {
    return __half22float2(*reinterpret_cast<__half2*>(&x));
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t x) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&x));
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void stsm_x4_t(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
    asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1,%2,%3,%4};"
                 :: "r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}
__device__ __forceinline__ void stsm_x4(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};"
                 :: "r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}
// D(16x8,f32) += A(16x16) * B(16x8); A row-major fragments, B column fragments.
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---- programmatic dependent launch: a kernel launched with the programmatic-stream-serialization attribute may start
//      while its predecessor in the stream is still running; it must call pdl_wait() before it touches anything the
//      predecessor writes. pdl_launch_dependents() in the predecessor lets the dependent grid be scheduled early. ----
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- mbarrier + bulk copy (TMA engine, untiled form) ----
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~a second (by default) and reports false (the caller records a status and unwinds).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int limit = (1 << 22)) {
    for (int i = 0; i < limit; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (i > 64) __nanosleep(64);
    }
    return false;
}
// global -> shared bulk copy; bytes multiple of 16, both addresses 16-byte aligned.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// shared -> global bulk copy (same alignment rules), tracked by the issuing thread's bulk-async groups
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 :: "l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all committed groups have finished READING shared memory (the buffers may be overwritten)
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all committed groups have completed
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// Chunk geometry. A "chunk" never straddles two sequences. For a packed batch the host supplies
// cu_seqlens [N+1] and chunk_indices [NT][2] = (sequence, chunk inside the sequence), the same
// tables the reference builds with prepare_chunk_indices; a fixed-length batch passes null tables.
// ---------------------------------------------------------------------------------------------
struct ChunkInfo {
    int seq;     // sequence index
    int row0;    // first token row in the flattened [B*T] token axis
    int valid;   // number of real tokens in this chunk (1..64)
};
__device__ __forceinline__ ChunkInfo chunk_info(int c, const int* cu_seqlens, const int* chunk_indices, int T) {
    ChunkInfo ci;
    if (cu_seqlens) {
        ci.seq = chunk_indices[2 * c];
        int lc = chunk_indices[2 * c + 1];
        int bos = cu_seqlens[ci.seq], eos = cu_seqlens[ci.seq + 1];
        ci.row0 = bos + lc * BT;
        ci.valid = min(BT, eos - ci.row0);
    } else {
        int cps = (T + BT - 1) / BT;
        ci.seq = c / cps;
        int lc = c - ci.seq * cps;
        ci.row0 = ci.seq * T + lc * BT;
        ci.valid = min(BT, T - lc * BT);
    }
    return ci;
}

}  // namespace kda
