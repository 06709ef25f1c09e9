// Chunk-parallel backward, gate-free part: per (chunk, head) the dense products that involve the carried
// states, as TF32 mma.sync GEMMs on fp32 operands staged in shared memory (value dimension in two halves):
//     dQg  = dO S^T                 dW = -dVn S^T              dKg = Vn dS'^T          [64 x 128]
//     dPs  = tril(dO Vn^T)          dAu = stril(dVn (beta V)^T)                         [64 x 64]
//     Zu   = A^T dVn  ->  dv = beta Zu (final, bf16),  dbeta_u = rowsum(Zu * V)
//     dD[k] = sum_v S[k,v] dS'[k,v]
// dQg, dW, dKg, dPs, dAu, dD, dbeta_u go to an fp32 scratch record per tile for the gated stage.
//
// Covers the state-dependent half of chunk_kda_bwd_kernel_wy_dqkg_fused (cula/kda/chunk_bwd.py:145-313) and the
// dAqk half of chunk_kda_bwd_kernel_dAv (cula/kda/chunk_bwd.py:63-125).
#include "kda_common.cuh"
#include "kda_params.h"

namespace kda {

constexpr int BD_THREADS = 512;
constexpr int BD_NQ = BD_THREADS / 128;   // column groups: a warp = 16-row tile x column group
constexpr int BD_NT128 = 128 / BD_NQ / 8; // n-tiles per warp over the 128 key channels
constexpr int BD_NT64 = 64 / BD_NQ / 8;   // n-tiles per warp over 64 token / value columns
constexpr int PR = 68;                    // padded fp32 row: fragment loads hit 32 distinct banks
// shared memory (floats)
constexpr int BD_S = 0;                   // S_h   [128][68]
constexpr int BD_DS = BD_S + 128 * PR;    // dS'_h [128][68]
constexpr int BD_DO = BD_DS + 128 * PR;   // dO_h  [64][68]
constexpr int BD_VN = BD_DO + 64 * PR;    // Vn_h
constexpr int BD_DVN = BD_VN + 64 * PR;   // dVn_h
constexpr int BD_V = BD_DVN + 64 * PR;    // V_h (raw)
constexpr int BD_A = BD_V + 64 * PR;      // A [64][68]
constexpr int BD_BETA = BD_A + 64 * PR;   // beta[64]
constexpr int BD_RED = BD_BETA + 64;      // dbeta_u partials [BD_NQ][64]
constexpr int BD_FLOATS = BD_RED + BD_NQ * 64;
constexpr int BD_SMEM = BD_FLOATS * 4;

// Round to tf32 (nearest, ties away from zero -- what cvt.rna.tf32.f32 does for finite values) with two integer
// instructions: add half an ulp of the 10-bit mantissa, clear the 13 low bits. The PTX conversion is emulated with
// about twice as many, and this kernel rounds tens of thousands of operands per tile.
__device__ __forceinline__ float tf32r(float x) {
    return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const float (&a)[4], float b0, float b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(__float_as_uint(a[0])), "r"(__float_as_uint(a[1])), "r"(__float_as_uint(a[2])), "r"(__float_as_uint(a[3])),
                   "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

// One (chunk, head) tile. next_tile >= 0 names the tile this CTA handles next: its inputs are pulled into L2 midway.
__device__ __forceinline__ void bd_tile(const BwdDenseParams& p, float* sm, const int tile, const int next_tile) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int mt = warp & 3, nh = warp >> 2;          // 16-row tile, column group
    const int c = tile / p.H, h = tile - c * p.H;
    const ChunkInfo ci = chunk_info(c, p.cu_seqlens, p.chunk_indices, p.T);
    const size_t tile_idx = (size_t)tile;
    const size_t tok_stride = (size_t)p.H * DV;
    const size_t base = (size_t)ci.row0 * tok_stride + (size_t)h * DV;
    const float gs = p.gscale[0], gs_inv = p.gscale[1];
    const float* Sg = p.h32 + tile_idx * (size_t)(DK * DV);
    const float* dSg = p.ds + tile_idx * (size_t)(DK * DV);
    const __half* Vng = reinterpret_cast<const __half*>(p.vnew) + tile_idx * (size_t)(BT * DV);
    const __half* dVng = reinterpret_cast<const __half*>(p.dvn) + tile_idx * (size_t)(BT * DV);
    const __nv_bfloat16* dOg = reinterpret_cast<const __nv_bfloat16*>(p.d_o);
    const __nv_bfloat16* Vg = reinterpret_cast<const __nv_bfloat16*>(p.v);
    float* scr = p.scratch + tile_idx * (size_t)BWD_SCRATCH_FLOATS;

    // A (fp32 [64][64]) and beta once. The staging loops are unrolled so that all loads of a thread are in flight
    // together (rolled, every iteration pays a full memory latency before its conversions and stores).
#pragma unroll
    for (int i = tid; i < 64 * 16; i += BD_THREADS) {
        const int row = i >> 4, c4 = (i & 15) * 4;
        const float4 a = *reinterpret_cast<const float4*>(p.akk + tile_idx * 4096 + row * 64 + c4);
        *reinterpret_cast<float4*>(sm + BD_A + row * PR + c4) = make_float4(tf32r(a.x), tf32r(a.y), tf32r(a.z), tf32r(a.w));
    }
    if (tid < 64) {
        float b = 0.f;
        if (tid < ci.valid) {
            size_t bi = (size_t)(ci.row0 + tid) * p.H + h;
            b = p.beta_fp32 ? reinterpret_cast<const float*>(p.beta)[bi]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.beta)[bi]);
            if (p.beta_logit) b = __fdividef(1.f, 1.f + __expf(-b));
        }
        sm[BD_BETA + tid] = b;
    }

    float accQ[BD_NT128][4], accW[BD_NT128][4], accK[BD_NT128][4], accP[BD_NT64][4], accA[BD_NT64][4];
#pragma unroll
    for (int i = 0; i < BD_NT128; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) accQ[i][e] = accW[i][e] = accK[i][e] = 0.f;
#pragma unroll
    for (int i = 0; i < BD_NT64; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) accP[i][e] = accA[i][e] = 0.f;
    float dD_part = 0.f, dbu0 = 0.f, dbu1 = 0.f;     // dD for row k = tid / BD_NQ (a column slice per thread); dbeta_u for rows 16mt+g, +8

    for (int vh = 0; vh < 2; ++vh) {
        __syncthreads();        // previous half's fragments are no longer read
        // ---- stage this value half ----
#pragma unroll
        for (int i = tid; i < 128 * 16; i += BD_THREADS) {
            const int row = i >> 4, c4 = (i & 15) * 4;
            const float4 a = *reinterpret_cast<const float4*>(Sg + row * DV + vh * 64 + c4);
            const float4 b = *reinterpret_cast<const float4*>(dSg + row * DV + vh * 64 + c4);
            *reinterpret_cast<float4*>(sm + BD_S + row * PR + c4) = make_float4(tf32r(a.x), tf32r(a.y), tf32r(a.z), tf32r(a.w));
            *reinterpret_cast<float4*>(sm + BD_DS + row * PR + c4) = make_float4(tf32r(b.x), tf32r(b.y), tf32r(b.z), tf32r(b.w));
        }
        for (int i = tid; i < 64 * 8; i += BD_THREADS) {
            const int row = i >> 3, c8 = (i & 7) * 8;
            uint4 ro = make_uint4(0, 0, 0, 0), rv = make_uint4(0, 0, 0, 0);
            if (row < ci.valid) {
                ro = *reinterpret_cast<const uint4*>(dOg + base + (size_t)row * tok_stride + vh * 64 + c8);
                rv = *reinterpret_cast<const uint4*>(Vg + base + (size_t)row * tok_stride + vh * 64 + c8);
            }
            const uint4 rn = *reinterpret_cast<const uint4*>(Vng + row * DV + vh * 64 + c8);
            const uint4 rd = *reinterpret_cast<const uint4*>(dVng + row * DV + vh * 64 + c8);
            const uint32_t wo[4] = {ro.x, ro.y, ro.z, ro.w}, wv[4] = {rv.x, rv.y, rv.z, rv.w};
            const uint32_t wn[4] = {rn.x, rn.y, rn.z, rn.w}, wd[4] = {rd.x, rd.y, rd.z, rd.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float2 f = unpack_bf16(wo[e]);
                sm[BD_DO + row * PR + c8 + 2 * e] = tf32r(gs * f.x);
                sm[BD_DO + row * PR + c8 + 2 * e + 1] = tf32r(gs * f.y);
                f = unpack_bf16(wv[e]);
                sm[BD_V + row * PR + c8 + 2 * e] = tf32r(f.x);
                sm[BD_V + row * PR + c8 + 2 * e + 1] = tf32r(f.y);
                f = unpack_f16(wn[e]);
                sm[BD_VN + row * PR + c8 + 2 * e] = tf32r(f.x);
                sm[BD_VN + row * PR + c8 + 2 * e + 1] = tf32r(f.y);
                f = unpack_f16(wd[e]);
                sm[BD_DVN + row * PR + c8 + 2 * e] = tf32r(f.x);
                sm[BD_DVN + row * PR + c8 + 2 * e + 1] = tf32r(f.y);
            }
        }
        __syncthreads();
        // next tile of this CTA: pull its inputs into L2 while the second half computes
        if (vh == 1 && next_tile >= 0) {
            const size_t nt_idx = (size_t)next_tile;
            const int cn = next_tile / p.H, hn = next_tile - cn * p.H;
            const ChunkInfo cin = chunk_info(cn, p.cu_seqlens, p.chunk_indices, p.T);
            const size_t nb = (size_t)cin.row0 * tok_stride + (size_t)hn * DV;
            for (int i = tid; i < 512; i += BD_THREADS) {     // S and dS': 64 KB each, 128-byte lines
                prefetch_l2(p.h32 + nt_idx * (size_t)(DK * DV) + 32 * i);
                prefetch_l2(p.ds + nt_idx * (size_t)(DK * DV) + 32 * i);
            }
            if (tid < 128) {
                prefetch_l2(reinterpret_cast<const __half*>(p.vnew) + nt_idx * (size_t)(BT * DV) + 64 * tid);
                prefetch_l2(reinterpret_cast<const __half*>(p.dvn) + nt_idx * (size_t)(BT * DV) + 64 * tid);
                prefetch_l2(p.akk + nt_idx * 4096 + 32 * tid);
            } else if (tid < 256) {
                const int row = (tid - 128) >> 1, half = tid & 1;
                if (row < cin.valid) {
                    prefetch_l2(dOg + nb + (size_t)row * tok_stride + 64 * half);
                    prefetch_l2(Vg + nb + (size_t)row * tok_stride + 64 * half);
                }
            }
        }
        // ---- dD partial: row k = tid ----
        {
            const int row = tid / BD_NQ, v0 = (tid % BD_NQ) * (64 / BD_NQ);
            float a = 0.f;
#pragma unroll 8
            for (int v = 0; v < 64 / BD_NQ; ++v) {
                const int vv = v0 + ((v + row) & (64 / BD_NQ - 1));      // rotated start: spreads the banks
                a = fmaf(sm[BD_S + row * PR + vv], sm[BD_DS + row * PR + vv], a);
            }
            dD_part += a;
        }
        // ---- contraction over the 64 value columns of this half ----
        // tf32 fragments come from ldmatrix: an 8 x 8 b16 tile is an 8 x 4 tile of 32-bit words, and lane l receives
        // word (row l / 4, column l % 4) -- exactly the m16n8k8 tf32 fragment layout. One x4 load fetches a whole
        // A fragment (rows 0-7 / 8-15 x words 0-3 / 4-7) or the B fragments of two n-tiles.
        const uint32_t sm_u32 = smem_u32(sm);
        const int lr = lane & 7, lm = lane >> 3;
        const uint32_t a_off = (uint32_t)(((16 * mt + lr + 8 * (lm & 1)) * PR + 4 * (lm >> 1)) * 4);   // + k0 * 4
        const uint32_t b_off = (uint32_t)(((lr + 8 * (lm >> 1)) * PR + 4 * (lm & 1)) * 4);              // + (n0 * PR + k0) * 4
#pragma unroll 2
        for (int ks = 0; ks < 8; ++ks) {
            const int k0 = 8 * ks;
            float fO[4], fV[4], fD[4];
            ldsm_x4(sm_u32 + BD_DO * 4 + a_off + k0 * 4, reinterpret_cast<uint32_t&>(fO[0]), reinterpret_cast<uint32_t&>(fO[1]),
                    reinterpret_cast<uint32_t&>(fO[2]), reinterpret_cast<uint32_t&>(fO[3]));
            ldsm_x4(sm_u32 + BD_VN * 4 + a_off + k0 * 4, reinterpret_cast<uint32_t&>(fV[0]), reinterpret_cast<uint32_t&>(fV[1]),
                    reinterpret_cast<uint32_t&>(fV[2]), reinterpret_cast<uint32_t&>(fV[3]));
            ldsm_x4(sm_u32 + BD_DVN * 4 + a_off + k0 * 4, reinterpret_cast<uint32_t&>(fD[0]), reinterpret_cast<uint32_t&>(fD[1]),
                    reinterpret_cast<uint32_t&>(fD[2]), reinterpret_cast<uint32_t&>(fD[3]));
#pragma unroll
            for (int np = 0; np < BD_NT128 / 2; ++np) {
                const int n0 = 8 * BD_NT128 * nh + 16 * np;      // key channels n0 .. n0 + 15
                float s[4], d[4];
                ldsm_x4(sm_u32 + (BD_S + n0 * PR + k0) * 4 + b_off, reinterpret_cast<uint32_t&>(s[0]), reinterpret_cast<uint32_t&>(s[1]),
                        reinterpret_cast<uint32_t&>(s[2]), reinterpret_cast<uint32_t&>(s[3]));
                ldsm_x4(sm_u32 + (BD_DS + n0 * PR + k0) * 4 + b_off, reinterpret_cast<uint32_t&>(d[0]), reinterpret_cast<uint32_t&>(d[1]),
                        reinterpret_cast<uint32_t&>(d[2]), reinterpret_cast<uint32_t&>(d[3]));
                mma_tf32(accQ[2 * np], fO, s[0], s[1]);
                mma_tf32(accW[2 * np], fD, s[0], s[1]);
                mma_tf32(accK[2 * np], fV, d[0], d[1]);
                mma_tf32(accQ[2 * np + 1], fO, s[2], s[3]);
                mma_tf32(accW[2 * np + 1], fD, s[2], s[3]);
                mma_tf32(accK[2 * np + 1], fV, d[2], d[3]);
            }
            static_assert(BD_NT64 == 2 && BD_NT128 % 2 == 0, "fragment pairing below assumes two token n-tiles per warp");
            {
                const int j0 = 8 * BD_NT64 * nh;                  // token columns j0 .. j0 + 15
                float vn[4], vv[4];
                ldsm_x4(sm_u32 + (BD_VN + j0 * PR + k0) * 4 + b_off, reinterpret_cast<uint32_t&>(vn[0]), reinterpret_cast<uint32_t&>(vn[1]),
                        reinterpret_cast<uint32_t&>(vn[2]), reinterpret_cast<uint32_t&>(vn[3]));
                ldsm_x4(sm_u32 + (BD_V + j0 * PR + k0) * 4 + b_off, reinterpret_cast<uint32_t&>(vv[0]), reinterpret_cast<uint32_t&>(vv[1]),
                        reinterpret_cast<uint32_t&>(vv[2]), reinterpret_cast<uint32_t&>(vv[3]));
                mma_tf32(accP[0], fO, vn[0], vn[1]);
                mma_tf32(accA[0], fD, vv[0], vv[1]);
                mma_tf32(accP[1], fO, vn[2], vn[3]);
                mma_tf32(accA[1], fD, vv[2], vv[3]);
            }
        }
        // ---- Zu = A^T dVn_h : [64 i] x [64 v of this half], contraction over the 64 tokens j ----
        float accZ[BD_NT64][4];
#pragma unroll
        for (int i = 0; i < BD_NT64; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) accZ[i][e] = 0.f;
#pragma unroll 2
        for (int ks = 0; ks < 8; ++ks) {
            const int j0 = 8 * ks, i0 = 16 * mt;
            const float fA[4] = {sm[BD_A + (j0 + t) * PR + i0 + g], sm[BD_A + (j0 + t) * PR + i0 + g + 8],
                                 sm[BD_A + (j0 + t + 4) * PR + i0 + g], sm[BD_A + (j0 + t + 4) * PR + i0 + g + 8]};
#pragma unroll
            for (int nt = 0; nt < BD_NT64; ++nt) {
                const int v0 = 8 * BD_NT64 * nh + 8 * nt;
                mma_tf32(accZ[nt], fA, sm[BD_DVN + (j0 + t) * PR + v0 + g], sm[BD_DVN + (j0 + t + 4) * PR + v0 + g]);
            }
        }
        {   // dv = beta * Zu (true units), dbeta_u += rowsum(Zu * V)
            const int r0 = 16 * mt + g, r1 = r0 + 8;
            const float b0 = sm[BD_BETA + r0], b1 = sm[BD_BETA + r1];
            __nv_bfloat16* dvp = reinterpret_cast<__nv_bfloat16*>(p.dv);
#pragma unroll
            for (int nt = 0; nt < BD_NT64; ++nt) {
                const int vc = 8 * BD_NT64 * nh + 8 * nt + 2 * t;
                dbu0 += accZ[nt][0] * sm[BD_V + r0 * PR + vc] + accZ[nt][1] * sm[BD_V + r0 * PR + vc + 1];
                dbu1 += accZ[nt][2] * sm[BD_V + r1 * PR + vc] + accZ[nt][3] * sm[BD_V + r1 * PR + vc + 1];
                if (r0 < ci.valid)
                    *reinterpret_cast<uint32_t*>(dvp + base + (size_t)r0 * tok_stride + vh * 64 + vc) =
                        pack_bf16(gs_inv * b0 * accZ[nt][0], gs_inv * b0 * accZ[nt][1]);
                if (r1 < ci.valid)
                    *reinterpret_cast<uint32_t*>(dvp + base + (size_t)r1 * tok_stride + vh * 64 + vc) =
                        pack_bf16(gs_inv * b1 * accZ[nt][2], gs_inv * b1 * accZ[nt][3]);
            }
        }
    }
    // ---- write the scratch record (units of gs) ----
    {
        const int r0 = 16 * mt + g, r1 = r0 + 8;
#pragma unroll
        for (int nt = 0; nt < BD_NT128; ++nt) {
            const int col = 8 * BD_NT128 * nh + 8 * nt + 2 * t;
            *reinterpret_cast<float2*>(scr + SCR_DQG + r0 * DK + col) = make_float2(accQ[nt][0], accQ[nt][1]);
            *reinterpret_cast<float2*>(scr + SCR_DQG + r1 * DK + col) = make_float2(accQ[nt][2], accQ[nt][3]);
            *reinterpret_cast<float2*>(scr + SCR_DW + r0 * DK + col) = make_float2(-accW[nt][0], -accW[nt][1]);
            *reinterpret_cast<float2*>(scr + SCR_DW + r1 * DK + col) = make_float2(-accW[nt][2], -accW[nt][3]);
            *reinterpret_cast<float2*>(scr + SCR_DKG + r0 * DK + col) = make_float2(accK[nt][0], accK[nt][1]);
            *reinterpret_cast<float2*>(scr + SCR_DKG + r1 * DK + col) = make_float2(accK[nt][2], accK[nt][3]);
        }
#pragma unroll
        for (int nt = 0; nt < BD_NT64; ++nt) {
            const int col = 8 * BD_NT64 * nh + 8 * nt + 2 * t;
            const float bj0 = sm[BD_BETA + col], bj1 = sm[BD_BETA + col + 1];
            float p00 = (col <= r0) ? accP[nt][0] : 0.f, p01 = (col + 1 <= r0) ? accP[nt][1] : 0.f;
            float p10 = (col <= r1) ? accP[nt][2] : 0.f, p11 = (col + 1 <= r1) ? accP[nt][3] : 0.f;
            float a00 = (col < r0) ? bj0 * accA[nt][0] : 0.f, a01 = (col + 1 < r0) ? bj1 * accA[nt][1] : 0.f;
            float a10 = (col < r1) ? bj0 * accA[nt][2] : 0.f, a11 = (col + 1 < r1) ? bj1 * accA[nt][3] : 0.f;
            *reinterpret_cast<float2*>(scr + SCR_DPS + r0 * BT + col) = make_float2(p00, p01);
            *reinterpret_cast<float2*>(scr + SCR_DPS + r1 * BT + col) = make_float2(p10, p11);
            *reinterpret_cast<float2*>(scr + SCR_DAU + r0 * BT + col) = make_float2(a00, a01);
            *reinterpret_cast<float2*>(scr + SCR_DAU + r1 * BT + col) = make_float2(a10, a11);
        }
        // dbeta_u: reduce over the 4 lanes of a quad, then over the column groups through shared memory
        dbu0 += __shfl_xor_sync(0xffffffffu, dbu0, 1); dbu0 += __shfl_xor_sync(0xffffffffu, dbu0, 2);
        dbu1 += __shfl_xor_sync(0xffffffffu, dbu1, 1); dbu1 += __shfl_xor_sync(0xffffffffu, dbu1, 2);
        if (t == 0) {
            sm[BD_RED + nh * 64 + r0] = dbu0;
            sm[BD_RED + nh * 64 + r1] = dbu1;
        }
        __syncthreads();
        if (tid < 64) {
            float v = 0.f;
#pragma unroll
            for (int x = 0; x < BD_NQ; ++x) v += sm[BD_RED + x * 64 + tid];
            scr[SCR_DBU + tid] = v;
        }
#pragma unroll
        for (int o = 1; o < BD_NQ; o <<= 1) dD_part += __shfl_xor_sync(0xffffffffu, dD_part, o);
        if (tid % BD_NQ == 0) scr[SCR_DD + tid / BD_NQ] = dD_part;
    }
}

// Persistent: CTA b handles tiles b, b + gridDim.x, ... so that the next tile's inputs can be prefetched.
__global__ void __launch_bounds__(BD_THREADS, 1) kda_bwd_dense_kernel(const BwdDenseParams p, const int num_tiles) {
    extern __shared__ __align__(16) float sm[];
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int next = tile + gridDim.x;
        bd_tile(p, sm, tile, next < num_tiles ? next : -1);
        __syncthreads();                                  // shared memory is reused by the next tile
    }
}

}  // namespace kda

extern "C" int kda_launch_bwd_dense(const kda::BwdDenseParams* p, int num_chunks, cudaStream_t stream) {
    using namespace kda;
    if (num_chunks <= 0) return 0;
    cudaError_t e = cudaFuncSetAttribute(kda_bwd_dense_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BD_SMEM);
    if (e != cudaSuccess) return (int)e;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = num_chunks * p->H;
    kda_bwd_dense_kernel<<<tiles < sms ? tiles : sms, BD_THREADS, BD_SMEM, stream>>>(*p, tiles);
    return (int)cudaGetLastError();
}
