// Chunk-parallel backward, gate-free part: per (chunk, head) the dense products that involve the carried states.
//     dQg  = dO S^T                 dW = -dVn S^T              dKg = Vn dS'^T          [64 x 128]
//     dPs  = tril(dO Vn^T)          dAu = stril(dVn (beta V)^T)                         [64 x 64]
//     Zu   = A^T dVn  ->  dv = beta Zu (final, bf16),  dbeta_u = rowsum(Zu * V)
//     dD[k] = sum_v S[k,v] dS'[k,v]
// dQg, dW, dKg, dPs, dAu, dD, dbeta_u go to an fp32 scratch record per tile for the gated stage.
//
// All products run on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory):
//   * the fp32 states S and dS' (64 KB each per tile, the bulk of the traffic) are fetched by the TMA engine through
//     tiled tensor maps (cp.async.bulk.tensor, 32 floats x 128 rows per box, 128-byte swizzle) straight into the
//     K-major operand layout of kind::tf32 -- no thread touches them except for the row sums of dD;
//   * the 16-bit operands (dO, V bf16; Vn, dVn fp16) are widened to 32-bit containers by the CUDA cores (every bf16 /
//     fp16 value is exact in tf32) and stacked so that ONE M = 128 instruction serves two products:
//         [dO; dVn] x S^T        -> TMEM lanes 0-63 dQg, lanes 64-127 -dW
//         [Vn; V ] x dS'^T       -> lanes 0-63 dKg
//         [dO; dVn] x [Vn; V]^T  -> lanes 0-63 / columns 0-63 dPs, lanes 64-127 / columns 64-127 the u-part of dA
//   * Zu = A^T dVn is a kind::f16 product with both operands MN-major (A and dVn are stored token-row-major and the
//     contraction runs over the token), A stacked twice so that both lane halves of TMEM hold Zu.
// The value dimension is processed in two halves that accumulate into the same TMEM columns; the TMA loads of both
// halves of the NEXT tile are in flight during the epilogue of this one, and the 16-bit operands of the next stage
// wait in registers. The tensor core truncates tf32 operands; the mean truncation error of the state operands is
// compensated by one factor in the epilogue. Every wait is bounded: on expiry the status word is set, the CTA waits
// (bounded) for its copies in flight, frees its tensor memory and returns.
//
// Covers the state-dependent half of chunk_kda_bwd_kernel_wy_dqkg_fused (cula/kda/chunk_bwd.py:145-313) and the
// dAqk half of chunk_kda_bwd_kernel_dAv (cula/kda/chunk_bwd.py:63-125).
#include <cuda.h>

#include "kda_common.cuh"
#include "kda_params.h"
#include "umma.cuh"

// Optional per-phase cycle counters (compile with -DKDA_PHASE_TIMERS): thread 0 of every CTA adds the clock64() spent
// between consecutive marks to a device array that kda_bwd_dense_read_timers() copies out (profiling builds only).
#ifdef KDA_PHASE_TIMERS
__device__ unsigned long long kda_bwd_dense_timers[16];
#define BD_MARK(i)                                                                        \
    do {                                                                                  \
        if (threadIdx.x == 0) {                                                           \
            const long long now_ = clock64();                                             \
            atomicAdd(&kda_bwd_dense_timers[i], (unsigned long long)(now_ - bd_t0_));     \
            bd_t0_ = now_;                                                                \
        }                                                                                 \
    } while (0)
#else
#define BD_MARK(i) do {} while (0)
#endif

namespace kda {

constexpr int BD_THREADS = 512;
// shared-memory map (bytes from a 1024-aligned base); an "atom" is [rows][128 B] with the 16-byte groups of a row
// XOR-swizzled by (row & 7) -- what the TMA engine writes with the 128-byte swizzle and what the MMA descriptors expect
constexpr int BD_S = 0;             // S   as B operand: [2 value halves][2 k-atoms][128 rows][128 B] fp32
constexpr int BD_DS = 65536;        // dS' likewise
constexpr int BD_A1 = 131072;       // [dO; dVn] of one value half: [2 k-atoms][128 rows][128 B] fp32
constexpr int BD_VNV = 163840;      // [Vn; V] of one value half, same shape
constexpr int BD_A4 = 196608;       // A fp16, stored twice: [2][64 tokens j][128 B] -- MN-major A operand of Zu
constexpr int BD_B4 = 212992;       // dVn fp16 of one value half: [64 tokens j][128 B] -- MN-major B operand of Zu
constexpr int BD_MISC = 221184;     // beta[64] f32 @0, dbeta_u partials [8][64] f32 @256, 4 mbarriers @2304, TMEM slot @2336, abort @2340
constexpr int BD_SMEM = BD_MISC + 2560 + 1024;
constexpr uint32_t BD_HALF_TX = 65536;   // bytes the TMA engine delivers per value half: 2 boxes of S + 2 of dS'
// TMEM columns
constexpr uint32_t TC_D1 = 0, TC_D2 = 128, TC_D3 = 256, TC_D4 = 384;
// mean relative truncation error of a tf32 operand with log-uniform mantissa is -2^-11 / ln 2; products with ONE
// truncated operand (the states) are scaled back by this factor
constexpr float TF32_TRUNC_COMP = 1.0003523f;

__device__ __forceinline__ uint64_t bd_sdesc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return umma::make_sdesc(addr, lbo, sbo) | (2ull << 61);     // 128-byte swizzle
}
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t smem_src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 :: "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_src), "r"(x), "r"(y), "r"(z) : "memory");
}
// byte offset of the 16-byte group `chunk` (0..7) of row `row` inside an atom
__device__ __forceinline__ uint32_t atom_off(int row, int chunk) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

struct BdStage {          // the 16-bit operands of one value half, as loaded: 8 consecutive value columns of one token row
    uint4 o, v, vn, dvn;
};

__global__ void __launch_bounds__(BD_THREADS, 1)
kda_bwd_dense_kernel(const BwdDenseParams p, const int num_tiles, const __grid_constant__ CUtensorMap map_s,
                     const __grid_constant__ CUtensorMap map_ds, const __grid_constant__ CUtensorMap map_out128,
                     const __grid_constant__ CUtensorMap map_out64) {
    extern __shared__ unsigned char bd_smem_raw[];
    unsigned char* sm = bd_smem_raw + ((1024u - (smem_u32(bd_smem_raw) & 1023u)) & 1023u);
    const uint32_t smb = smem_u32(sm);
    float* sBeta = reinterpret_cast<float*>(sm + BD_MISC);
    float* sRed = reinterpret_cast<float*>(sm + BD_MISC + 256);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + BD_MISC + 2304);    // [0,1] states of half 0 / 1 landed; [2,3] MMAs of half 0 / 1 done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + BD_MISC + 2336);
    volatile int* sAbort = reinterpret_cast<volatile int*>(sm + BD_MISC + 2340);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t tok_stride = (size_t)p.H * DV;
    const float gs = p.gscale[0], gs_inv = p.gscale[1];
    const __nv_bfloat16* dOg = reinterpret_cast<const __nv_bfloat16*>(p.d_o);
    const __nv_bfloat16* Vg = reinterpret_cast<const __nv_bfloat16*>(p.v);
    // staging role: token row and 8 value columns (of the 64 of a half)
    const int srow = tid >> 3, sc8 = tid & 7;

    if (tid == 0) {
        for (int i = 0; i < 4; ++i) mbar_init(&bars[i], 1);
        *sAbort = 0;
        fence_mbar_init();
    }
    if (warp == 0) umma::tmem_alloc(tmem_slot, 512);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    // ---- helpers ----
    auto issue_state_loads = [&](int t_id, int vh) {        // one thread: one value half of S and dS' of a tile
        mbar_arrive_expect_tx(&bars[vh], BD_HALF_TX);
#pragma unroll
        for (int a = 0; a < 2; ++a) {
            tma_load_2d(smb + BD_S + vh * 32768 + a * 16384, &map_s, vh * 64 + a * 32, t_id * 128, &bars[vh]);
            tma_load_2d(smb + BD_DS + vh * 32768 + a * 16384, &map_ds, vh * 64 + a * 32, t_id * 128, &bars[vh]);
        }
    };
    auto fetch_stage = [&](int t_id, const ChunkInfo& ci, int h, int vh) -> BdStage {
        BdStage s;
        const int row = min(srow, ci.valid - 1);     // a padding row re-reads the last real row and is zeroed below
        const size_t goff = (size_t)(ci.row0 + row) * tok_stride + (size_t)h * DV + vh * 64 + sc8 * 8;
        s.o = *reinterpret_cast<const uint4*>(dOg + goff);
        s.v = *reinterpret_cast<const uint4*>(Vg + goff);
        const size_t toff = (size_t)t_id * (BT * DV) + srow * DV + vh * 64 + sc8 * 8;
        s.vn = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.vnew) + toff);
        s.dvn = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.dvn) + toff);
        return s;
    };
    // widen 8 values to fp32 and store them as two 16-byte groups of an fp32 K-major atom pair
    auto put8 = [&](int base, int row, float scale, const uint4& raw, bool is_bf16) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        float f[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 x = is_bf16 ? unpack_bf16(w[e]) : unpack_f16(w[e]);
            f[2 * e] = scale * x.x;
            f[2 * e + 1] = scale * x.y;
        }
        unsigned char* atom = sm + base + (sc8 >> 2) * 16384;
        const int ch = (sc8 & 3) * 2;
        *reinterpret_cast<float4*>(atom + atom_off(row, ch)) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(atom + atom_off(row, ch + 1)) = make_float4(f[4], f[5], f[6], f[7]);
    };
    auto store_stage = [&](const BdStage& s, bool real_row) {
        put8(BD_A1, srow, real_row ? gs : 0.f, s.o, true);          // dO (units of the gradient scale)
        put8(BD_A1, srow + 64, 1.f, s.dvn, false);                   // dVn
        put8(BD_VNV, srow, 1.f, s.vn, false);                        // Vn
        put8(BD_VNV, srow + 64, real_row ? 1.f : 0.f, s.v, true);    // V
        *reinterpret_cast<uint4*>(sm + BD_B4 + atom_off(srow, sc8)) = s.dvn;
    };
    // One thread waits (bounded) for an mbarrier; everybody else parks on the CTA barrier.
    auto cta_wait = [&](int which, uint32_t parity) -> bool {
        if (tid == 0) {
            if (!*sAbort && !mbar_wait(&bars[which], parity)) {
                atomicExch(p.status, STATUS_WAIT_TIMEOUT);
                *sAbort = 1;
            }
            umma::fence_before_sync();
        }
        __syncthreads();
        umma::fence_after_sync();
        return *sAbort == 0;
    };

    // ---- prologue: first tile's loads ----
    int tile = blockIdx.x;
    int h = 0;
    ChunkInfo ci{};
    BdStage st{};
    float4 a_lo = make_float4(0, 0, 0, 0), a_hi = a_lo;
    uint32_t beta_raw = 0;
    auto fetch_tile_top = [&](int t_id) {       // geometry, A, beta (raw bits) and the first value half of a tile
        const int c = t_id / p.H;
        h = t_id - c * p.H;
        ci = chunk_info(c, p.cu_seqlens, p.chunk_indices, p.T);
        st = fetch_stage(t_id, ci, h, 0);
        const float* ag = p.akk + (size_t)t_id * 4096 + srow * 64 + sc8 * 8;
        a_lo = *reinterpret_cast<const float4*>(ag);
        a_hi = *reinterpret_cast<const float4*>(ag + 4);
        if (tid < 64) {
            const size_t bi = (size_t)(ci.row0 + min(tid, ci.valid - 1)) * p.H + h;
            beta_raw = p.beta_fp32 ? reinterpret_cast<const uint32_t*>(p.beta)[bi]
                                   : (uint32_t)reinterpret_cast<const unsigned short*>(p.beta)[bi] << 16;
        }
    };
    bool issued1 = false;                       // thread 0: the loads of value half 1 of the current tile have been issued
    if (tile < num_tiles) {
        if (tid == 0) {
            issue_state_loads(tile, 0);
            issue_state_loads(tile, 1);
            issued1 = true;
        }
        fetch_tile_top(tile);
    }

    const uint32_t idesc_tf32 = umma::make_idesc(umma::FMT_TF32, 128, 128, false, false);
    const uint32_t idesc_zu = umma::make_idesc(umma::FMT_F16, 128, 64, true, true);
    uint32_t par = 0;
    // dD role (warps 1-15; warp 0 issues the MMAs instead): item = (state row k, 16-byte group) of 1024 per value half
    const int dd_idx = tid - 32;

#ifdef KDA_PHASE_TIMERS
    long long bd_t0_ = clock64();
#endif
    for (; tile < num_tiles; tile += gridDim.x, par ^= 1u) {
        const int next = tile + gridDim.x;
        const ChunkInfo cur = ci;
        const int cur_h = h;
        float dD_part[3] = {0.f, 0.f, 0.f};
        // ---- stage A, beta and the first value half. The previous tile's MMAs have completed and its first group of
        //      output stores has been read out of the staging buffers (checked before its last barrier) ----
        {
            const uint4 a16 = make_uint4(pack_f16(a_lo.x, a_lo.y), pack_f16(a_lo.z, a_lo.w), pack_f16(a_hi.x, a_hi.y),
                                         pack_f16(a_hi.z, a_hi.w));
            *reinterpret_cast<uint4*>(sm + BD_A4 + atom_off(srow, sc8)) = a16;
            *reinterpret_cast<uint4*>(sm + BD_A4 + 8192 + atom_off(srow, sc8)) = a16;
            if (tid < 64) {
                float b = __uint_as_float(beta_raw);
                if (p.beta_logit) b = __fdividef(1.f, 1.f + __expf(-b));
                sBeta[tid] = tid < cur.valid ? b : 0.f;
            }
        }
#pragma unroll 1
        for (int vh = 0; vh < 2; ++vh) {
            store_stage(st, srow < cur.valid);
            fence_proxy_async();
            __syncthreads();
            BD_MARK(0 + 6 * vh);      // operands widened into shared memory
            // operands of the next stage into registers: the second half of this tile, or the top of the next tile (its
            // geometry costs a few hundred instructions: the issuing thread does this after the MMAs are on their way)
            auto fetch_next = [&]() {
                if (vh == 0) st = fetch_stage(tile, cur, cur_h, 1);
                else if (next < num_tiles) fetch_tile_top(next);
            };
            if (warp != 0 || vh == 0) fetch_next();
            BD_MARK(1 + 6 * vh);
            // ---- one thread: wait for the states of this half, issue the MMAs ----
            if (tid == 0) {
                if (vh == 0 && !issued1) {
                    // the second output group of the previous tile was staged in the half-1 state buffers
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    issue_state_loads(tile, 1);
                    issued1 = true;
                }
                if (!mbar_wait(&bars[vh], par)) {
                    atomicExch(p.status, STATUS_WAIT_TIMEOUT);
                    *sAbort = 1;
                } else {
                    BD_MARK(2 + 6 * vh);      // wait for the states of this half
                    umma::fence_after_sync();
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint32_t koff = (uint32_t)((ks >> 2) * 16384 + (ks & 3) * 32);
                        const uint64_t a1 = bd_sdesc(smb + BD_A1 + koff, 16, 1024);
                        const uint64_t vnv = bd_sdesc(smb + BD_VNV + koff, 16, 1024);
                        const uint64_t sd = bd_sdesc(smb + BD_S + vh * 32768 + koff, 16, 1024);
                        const uint64_t dsd = bd_sdesc(smb + BD_DS + vh * 32768 + koff, 16, 1024);
                        const uint32_t acc = (vh | ks) != 0;
                        umma::mma_tf32(tmem + TC_D1, a1, sd, idesc_tf32, acc);
                        umma::mma_tf32(tmem + TC_D2, vnv, dsd, idesc_tf32, acc);
                        umma::mma_tf32(tmem + TC_D3, a1, vnv, idesc_tf32, acc);
                    }
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t a4 = bd_sdesc(smb + BD_A4 + ks * 2048, 8192, 1024);
                        const uint64_t b4 = bd_sdesc(smb + BD_B4 + ks * 2048, 8192, 1024);
                        umma::mma_f16(tmem + TC_D4 + vh * 64, a4, b4, idesc_zu, ks != 0);
                    }
                    umma::commit(&bars[2 + vh]);
                    BD_MARK(3 + 6 * vh);      // MMA issue
                }
            } else if (warp != 0) {
                // ---- dD partial of this half from the fp32 states in shared memory, under the MMAs ----
                if (!mbar_wait(&bars[vh], par)) {
                    atomicExch(p.status, STATUS_WAIT_TIMEOUT);
                    *sAbort = 1;
                }
#pragma unroll
                for (int n = 0; n < 3; ++n) {
                    const int item = dd_idx + 480 * n;
                    if (item < 1024) {
                        const int k = item >> 3;
                        const uint32_t off = vh * 32768 + atom_off(k, item & 7);
                        float acc = 0.f;
#pragma unroll
                        for (int a = 0; a < 2; ++a) {
                            const float4 x = *reinterpret_cast<const float4*>(sm + BD_S + a * 16384 + off);
                            const float4 y = *reinterpret_cast<const float4*>(sm + BD_DS + a * 16384 + off);
                            acc = fmaf(x.x, y.x, fmaf(x.y, y.y, fmaf(x.z, y.z, fmaf(x.w, y.w, acc))));
                        }
                        dD_part[n] += acc;
                    }
                }
            }
            if (warp == 0 && vh == 1) fetch_next();
            BD_MARK(4 + 6 * vh);          // thread 0: next operands requested
            if (!cta_wait(2 + vh, par)) break;
            BD_MARK(5 + 6 * vh);          // wait for the MMAs
        }
        if (*sAbort) break;
        // ---- the half-0 state buffers are free: the next tile's first loads run under the epilogue ----
        if (tid == 0) {
            issued1 = false;
            if (next < num_tiles) issue_state_loads(next, 0);
        }
        // ---- epilogue: TMEM -> registers -> swizzled staging buffers -> TMA tensor stores into the scratch record ----
        {
            float* scr = p.scratch + (size_t)tile * BWD_SCRATCH_FLOATS;
            const int q = warp & 3, cg = warp >> 2;
            const int i = 32 * (q & 1) + lane;                       // token row of this thread
            const bool upper = q < 2;                                // TMEM lanes 0-63
            const uint32_t tl = tmem + ((uint32_t)(32 * q) << 16);
            uint32_t r[16];
            // D1: dQg (lanes 0-63) / -dW (lanes 64-127), 32 of the 128 key channels per warp -> boxes in the [dO; dVn] / [Vn; V] buffers
            {
                unsigned char* box = sm + BD_A1 + ((upper ? 0 : 4) + cg) * 8192;
                const float f = upper ? TF32_TRUNC_COMP : -TF32_TRUNC_COMP;
#pragma unroll
                for (int part = 0; part < 2; ++part) {
                    umma::ld_32x32b_x16(tl + TC_D1 + 32 * cg + 16 * part, r);
                    umma::wait_ld();
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        *reinterpret_cast<float4*>(box + atom_off(i, 4 * part + e)) =
                            make_float4(f * __uint_as_float(r[4 * e]), f * __uint_as_float(r[4 * e + 1]),
                                        f * __uint_as_float(r[4 * e + 2]), f * __uint_as_float(r[4 * e + 3]));
                }
            }
            fence_proxy_async();
            __syncthreads();
            if (tid == 0) {
#pragma unroll
                for (int b = 0; b < 8; ++b)
                    tma_store_3d(&map_out128, smb + BD_A1 + b * 8192, 32 * (b & 3), 64 * (b >> 2), tile);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            BD_MARK(12);                  // dQg, dW staged and their stores issued
            // D2: dKg (lanes 0-63 only) -> boxes in the half-1 buffer of S
            if (upper) {
                unsigned char* box = sm + BD_S + 32768 + cg * 8192;
#pragma unroll
                for (int part = 0; part < 2; ++part) {
                    umma::ld_32x32b_x16(tl + TC_D2 + 32 * cg + 16 * part, r);
                    umma::wait_ld();
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        *reinterpret_cast<float4*>(box + atom_off(i, 4 * part + e)) =
                            make_float4(TF32_TRUNC_COMP * __uint_as_float(r[4 * e]), TF32_TRUNC_COMP * __uint_as_float(r[4 * e + 1]),
                                        TF32_TRUNC_COMP * __uint_as_float(r[4 * e + 2]), TF32_TRUNC_COMP * __uint_as_float(r[4 * e + 3]));
                }
            }
            // D3: dPs = tril(dO Vn^T) (lanes 0-63, columns 0-63) / dAu = stril(dVn V^T) beta_j (lanes 64-127, columns 64-127)
            //     -> boxes in the half-1 buffer of dS'
            {
                const int j0 = 16 * cg;
                umma::ld_32x32b_x16(tl + TC_D3 + (upper ? 0 : 64) + j0, r);
                umma::wait_ld();
                unsigned char* box = sm + BD_DS + 32768 + ((upper ? 0 : 2) + (cg >> 1)) * 8192;
                float o[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int j = j0 + e;
                    const float x = __uint_as_float(r[e]);
                    o[e] = upper ? (j <= i ? x : 0.f) : (j < i ? sBeta[j] * x : 0.f);
                }
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    *reinterpret_cast<float4*>(box + atom_off(i, (cg & 1) * 4 + e)) = make_float4(o[4 * e], o[4 * e + 1], o[4 * e + 2], o[4 * e + 3]);
            }
            // D4: Zu (both lane halves hold it): lanes 0-63 take value columns 0-63, lanes 64-127 columns 64-127
            {
                const int v0 = (upper ? 0 : 64) + 16 * cg;
                umma::ld_32x32b_x16(tl + TC_D4 + v0, r);
                umma::wait_ld();
                float dbu = 0.f;
                if (i < cur.valid) {
                    const size_t goff = (size_t)(cur.row0 + i) * tok_stride + (size_t)cur_h * DV + v0;
                    const uint4 v_lo = *reinterpret_cast<const uint4*>(Vg + goff);
                    const uint4 v_hi = *reinterpret_cast<const uint4*>(Vg + goff + 8);
                    const uint32_t vw[8] = {v_lo.x, v_lo.y, v_lo.z, v_lo.w, v_hi.x, v_hi.y, v_hi.z, v_hi.w};
                    const float bsc = gs_inv * sBeta[i];
                    uint32_t out[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float2 vv = unpack_bf16(vw[e]);
                        const float z0 = __uint_as_float(r[2 * e]), z1 = __uint_as_float(r[2 * e + 1]);
                        dbu = fmaf(z0, vv.x, fmaf(z1, vv.y, dbu));
                        out[e] = pack_bf16(bsc * z0, bsc * z1);
                    }
                    __nv_bfloat16* dvp = reinterpret_cast<__nv_bfloat16*>(p.dv) + goff;
                    *reinterpret_cast<uint4*>(dvp) = make_uint4(out[0], out[1], out[2], out[3]);
                    *reinterpret_cast<uint4*>(dvp + 8) = make_uint4(out[4], out[5], out[6], out[7]);
                }
                sRed[((upper ? 0 : 4) + cg) * 64 + i] = dbu;
            }
            // dD: the eight 16-byte groups of a state row sit in adjacent lanes
            if (warp != 0) {
#pragma unroll
                for (int n = 0; n < 3; ++n) {
                    const int item = dd_idx + 480 * n;
                    if (item < 1024) {            // uniform per warp
                        float v = dD_part[n];
                        v += __shfl_xor_sync(0xffffffffu, v, 1);
                        v += __shfl_xor_sync(0xffffffffu, v, 2);
                        v += __shfl_xor_sync(0xffffffffu, v, 4);
                        if ((item & 7) == 0) scr[SCR_DD + (item >> 3)] = v;
                    }
                }
            }
            BD_MARK(13);                  // dKg, dPs, dAu staged; dv stored
            // the first group of stores must have been read out before the next tile's operands overwrite its buffers
            if (tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            fence_proxy_async();
            umma::fence_before_sync();
            __syncthreads();          // TMEM, the staging buffers and the dbeta_u partials are complete / free
            umma::fence_after_sync();
            if (tid == 0) {
#pragma unroll
                for (int b = 0; b < 4; ++b) tma_store_3d(&map_out128, smb + BD_S + 32768 + b * 8192, 32 * b, 128, tile);
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    tma_store_3d(&map_out64, smb + BD_DS + 32768 + b * 8192, 32 * (b & 1), 64 * (b >> 1), tile);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            if (tid < 64) {
                float v = 0.f;
#pragma unroll
                for (int x = 0; x < 8; ++x) v += sRed[x * 64 + tid];
                scr[SCR_DBU + tid] = v;
            }
        }
        BD_MARK(14);                      // end-of-tile barrier, second group of stores issued
    }
    // ---- unwind: copies in flight must land / be read out before the CTA's shared memory goes away ----
    if (tid == 0) {
        if (*sAbort) {
            mbar_wait(&bars[0], par);
            if (issued1) mbar_wait(&bars[1], par);
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, 512);
}

}  // namespace kda

#ifdef KDA_PHASE_TIMERS
extern "C" int kda_bwd_dense_read_timers(unsigned long long* out, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out, kda_bwd_dense_timers, sizeof(kda_bwd_dense_timers));
    if (e == cudaSuccess && reset) {
        unsigned long long z[16] = {};
        e = cudaMemcpyToSymbol(kda_bwd_dense_timers, z, sizeof(z));
    }
    return (int)e;
}
#endif

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// fp32 [tiles * 128 rows][128 columns], fetched as boxes of 32 columns x 128 rows with the 128-byte swizzle
bool make_state_map(CUtensorMap* map, const float* base, int tiles) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {128, (cuuint64_t)tiles * 128};
    const cuuint64_t strides[1] = {128 * sizeof(float)};
    const cuuint32_t box[2] = {32, 128};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The scratch record as a rank-3 tensor [tiles][rows][cols] of fp32, stored from boxes of 32 columns x 64 rows with the
// 128-byte swizzle. first_float: offset of the first matrix inside a record; rows: number of 64-row matrices x 64.
bool make_scratch_map(CUtensorMap* map, float* scratch, int first_float, int cols, int rows, int tiles) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)tiles};
    const cuuint64_t strides[2] = {cols * sizeof(float), kda::BWD_SCRATCH_FLOATS * sizeof(float)};
    const cuuint32_t box[3] = {32, 64, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, scratch + first_float, dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" int kda_launch_bwd_dense(const kda::BwdDenseParams* p, int num_chunks, cudaStream_t stream) {
    using namespace kda;
    if (num_chunks <= 0) return 0;
    cudaError_t e = cudaFuncSetAttribute(kda_bwd_dense_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BD_SMEM);
    if (e != cudaSuccess) return (int)e;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = num_chunks * p->H;
    static_assert(SCR_DW == SCR_DQG + 64 * 128 && SCR_DKG == SCR_DW + 64 * 128 && SCR_DAU == SCR_DPS + 64 * 64,
                  "the tensor maps below address dQg | dW | dKg and dPs | dAu as stacked matrices");
    static_assert((BWD_SCRATCH_FLOATS * 4) % 16 == 0 && (SCR_DPS * 4) % 16 == 0, "TMA strides and bases are 16-byte multiples");
    CUtensorMap map_s, map_ds, map_out128, map_out64;
    if (!make_state_map(&map_s, p->h32, tiles) || !make_state_map(&map_ds, p->ds, tiles) ||
        !make_scratch_map(&map_out128, p->scratch, SCR_DQG, 128, 192, tiles) ||
        !make_scratch_map(&map_out64, p->scratch, SCR_DPS, 64, 128, tiles))
        return (int)cudaErrorInvalidValue;
    kda_bwd_dense_kernel<<<tiles < sms ? tiles : sms, BD_THREADS, BD_SMEM, stream>>>(*p, tiles, map_s, map_ds, map_out128,
                                                                                      map_out64);
    return (int)cudaGetLastError();
}
