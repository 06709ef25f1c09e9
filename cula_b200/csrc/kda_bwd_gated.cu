// Chunk-parallel backward, gated part: per (chunk, head), from the scratch record of the dense stage,
//   dA  = dAu + stril(dW X^T),  dL = -stril(A^T dA A^T),  Zw = A^T dW  (gradient w.r.t. X = beta k 2^g)
//   VJPs of the two gated Gram matrices (Aqk and L), chain rule to q-hat, k-hat and the cumulative gate,
//   reverse cumulative sum, gate activation VJP (dg, dA_log, d dt_bias), L2-norm VJP; dq, dk, dg, dbeta to HBM.
//
// Covers the gate-dependent half of chunk_kda_bwd_kernel_wy_dqkg_fused (cula/kda/chunk_bwd.py:145-313),
// chunk_kda_bwd_kernel_intra (cula/kda/chunk_intra.py:367-627), the reverse chunk_local_cumsum and
// kda_gate_bwd (cula/kda/chunk_bwd.py:594-602) and l2norm_bwd (cula/kda/chunk.py:190-192).
//
// All contractions run as TF32 mma.sync (m16n8k8) on fp32 operands in shared memory. The Gram-matrix VJPs
//     dq_i += sum_{j<=i} cP_ij k_j 2^(g_i-g_j)        dk_i += sum_{j<i} cR_ij k_j 2^(g_i-g_j)
//     dk_j += sum_{i>=j} (cP_ij q_i + cR_ij k_i) 2^(g_i-g_j)
// never form 2^(g_i-g_j) pairwise: for the rows of a 16-row block I the column operand is k_j 2^(r_I-g_j)
// (r_I = g at the first row of the block, generated on the fly inside the B fragments) and the result is
// rescaled by 2^(g_i-r_I); for the columns of block J the row operands are q_i, k_i times 2^(g_i-s_J)
// (s_J = g at the last row of the block) and the result is rescaled by 2^(s_J-g_j). Every factor is either
// <= 1 or bounded by 2^(15*5*log2 e) ~ 2^108 under the safe gate, and the large ones only meet zero coefficients.
#include "kda_common.cuh"
#include "kda_params.h"

// Optional per-phase cycle counters (compile with -DKDA_PHASE_TIMERS): thread 0 of every CTA adds the clock64() spent
// between consecutive marks to a device array that kda_bwd_gated_read_timers() copies out (profiling builds only).
#ifdef KDA_PHASE_TIMERS
__device__ unsigned long long kda_bwd_gated_timers[16];
#define BG_MARK(i)                                                                        \
    do {                                                                                  \
        if (threadIdx.x == 0) {                                                           \
            const long long now_ = clock64();                                             \
            atomicAdd(&kda_bwd_gated_timers[i], (unsigned long long)(now_ - bg_t0_));     \
            bg_t0_ = now_;                                                                \
        }                                                                                 \
    } while (0)
#else
#define BG_MARK(i) do {} while (0)
#endif

namespace kda {

constexpr int BG_THREADS = 512;
constexpr int BG_WARPS = BG_THREADS / 32;
constexpr int BG_NQ = BG_WARPS / 4;              // column groups in the GEMM phases (a warp = 16-row tile x column group)
constexpr int BG_NT64 = 64 / BG_NQ / 8;          // n-tiles per warp over 64 columns
constexpr int BG_NT128 = 128 / BG_NQ / 8;        // n-tiles per warp over 128 columns
constexpr int BG_NT6 = 128 / BG_WARPS / 8;       // n-tiles per warp in the Gram VJPs (a warp owns 128 / BG_WARPS channels)
constexpr int BG_PASS_ROWS = BG_THREADS / 16;    // rows per pass of the wide loads (16 threads per row)
constexpr int BG_SEG = BG_THREADS / 128;         // row segments of the cumulative sums (a thread per channel and segment)
constexpr int BG_SEG_ROWS = 64 / BG_SEG;
constexpr int AR = 68;                         // padded row of the 64x64 fp32 matrices
constexpr int AS = 136;                        // padded row of the 64x128 fp32 matrices: both fragment patterns
                                               // (8 rows x 4 columns, 4 rows x 8 columns) hit 32 distinct banks
constexpr int GS = 136;                        // row of the gate matrix (floats), same reason
constexpr int QS = 136;                        // row of the bf16 q / k copies (elements): 68 words
// shared memory map (floats)
constexpr int BG_G = 0;                        // G    [64][128] log2 cumulative gate
constexpr int BG_ACC1 = BG_G + 64 * GS;           // dW, later dq-hat accumulator            [64][132]
constexpr int BG_ACC2 = BG_ACC1 + 64 * AS;     // dk-hat accumulator
constexpr int BG_ACC3 = BG_ACC2 + 64 * AS;     // X, later dG accumulator
constexpr int BG_QK = BG_ACC3 + 64 * AS;       // q raw, k raw as bf16 [64][QS] each
constexpr int BG_A = BG_QK + 64 * QS;             // A [64][68]
constexpr int BG_C1 = BG_A + 64 * AR;          // T1, later cP = scale * dPs          [64][68]
constexpr int BG_C2 = BG_C1 + 64 * AR;         // dA, later cR = beta_i * dL          [64][68]
constexpr int BG_MISC = BG_C2 + 64 * AR;
constexpr int MS_RSTDQ = 0, MS_RSTDK = 64, MS_BETA = 128, MS_DBETA = 192, MS_RED = 256 /* [BG_WARPS] */,
              MS_PBETA = 288 /* [BG_NQ][64] */, MS_PGL = MS_PBETA + BG_NQ * 64 /* [4][128] */,
              MS_HALF = MS_PGL /* [BG_SEG][128], used before and after the lifetime of MS_PGL */,
              MS_COL = MS_PGL + 512 /* [128] */, MS_END = MS_COL + 128;
static_assert(BG_SEG <= 4, "segment totals share the 512 floats of MS_PGL");
constexpr int BG_FLOATS = BG_MISC + MS_END;
constexpr int BG_SMEM = BG_FLOATS * 4;

// Round to tf32 (nearest, ties away from zero -- what cvt.rna.tf32.f32 does for finite values) with two integer
// instructions: add half an ulp of the 10-bit mantissa, clear the 13 low bits. The PTX conversion is emulated with
// about twice as many, and this kernel rounds tens of thousands of operands per tile.
__device__ __forceinline__ float bg_tf32(float x) {
    return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}
__device__ __forceinline__ void bg_mma(float (&d)[4], const float (&a)[4], float b0, float b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(__float_as_uint(a[0])), "r"(__float_as_uint(a[1])), "r"(__float_as_uint(a[2])), "r"(__float_as_uint(a[3])),
                   "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}
// The same with the B operand carried as a tf32 hi/lo pair (two MMAs): B is then exact to ~2^-22. Used for the Gram
// VJPs, where every pair (i, j) adds +x to the gate gradient of row i and -x to that of row j through two different
// products; the reverse cumulative sum relies on those two cancelling, so they must agree far better than tf32.
__device__ __forceinline__ float bg_tf32_lo(float x) {      // the low part of a split: truncation is enough (error 2^-21 of the value)
    return __uint_as_float(__float_as_uint(x) & 0xffffe000u);
}
__device__ __forceinline__ void bg_mma_split(float (&d)[4], const float (&a)[4], float b0, float b1) {
    const float h0 = bg_tf32(b0), h1 = bg_tf32(b1);
    bg_mma(d, a, bg_tf32_lo(b0 - h0), bg_tf32_lo(b1 - h1));
    bg_mma(d, a, h0, h1);
}
// natural-log decay a(x) of one raw gate value and (optionally) da/dx and the A_log-gradient integrand
__device__ __forceinline__ float bg_gate(float graw, float bias, float alpha, int mode, float lb) {
    if (mode == GATE_NONE) return graw;
    const float x = graw + bias;
    if (mode == GATE_LOWER_BOUND) return lb * fast_rcp(1.f + fast_exp2(-alpha * RCP_LN2 * x));
    return -alpha * (x > 20.f ? x : log1pf(__expf(x)));
}

// One (chunk, head) tile. next_tile >= 0 names the tile this CTA handles next: its inputs are pulled into L2 midway.
__device__ __forceinline__ void bg_tile(const BwdGatedParams& p, float* sm, const int tile, const int next_tile) {
    float* sG = sm + BG_G;
    float* acc1 = sm + BG_ACC1;
    float* acc2 = sm + BG_ACC2;
    float* acc3 = sm + BG_ACC3;
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(sm + BG_QK);
    __nv_bfloat16* sK = sQ + 64 * QS;
    float* sA = sm + BG_A;
    float* c1 = sm + BG_C1;
    float* c2 = sm + BG_C2;
    float* misc = sm + BG_MISC;
    float* rstd_q = misc + MS_RSTDQ;
    float* rstd_k = misc + MS_RSTDK;
    float* sBeta = misc + MS_BETA;
    float* sDbeta = misc + MS_DBETA;
    float* sHalf = misc + MS_HALF;
    float* sRed = misc + MS_RED;
    float* pBeta = misc + MS_PBETA;
    float* pGl = misc + MS_PGL;
    float* sCol = misc + MS_COL;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g8 = lane >> 2, t4 = lane & 3;
#ifdef KDA_PHASE_TIMERS
    long long bg_t0_ = clock64();
#endif
    const int c = tile / p.H, h = tile - c * p.H;
    const ChunkInfo ci = chunk_info(c, p.cu_seqlens, p.chunk_indices, p.T);
    const size_t tile_idx = (size_t)tile;
    const size_t tok_stride = (size_t)p.H * DK;
    const size_t base = (size_t)ci.row0 * tok_stride + (size_t)h * DK;
    const float* scr = p.scratch + tile_idx * (size_t)BWD_SCRATCH_FLOATS;
    const float gs_inv = p.gscale[1];
    const float alpha = p.gate_mode != GATE_NONE ? __expf(p.A_log[h]) : 0.f;
    const int pc = tid & 15;
    float bias[8];
#pragma unroll
    for (int e = 0; e < 8; ++e)
        bias[e] = (p.gate_mode != GATE_NONE && p.dt_bias) ? p.dt_bias[h * DK + 64 * (e >> 2) + 4 * pc + (e & 3)] : 0.f;

    // ---- 1a. wide loads: gate activation -> sG (log2 domain, zero for padding rows); q, k -> bf16 copies + norms.
    //          All global loads of the two passes are issued before the first use (a load that is consumed right away
    //          costs a full memory latency per pass); a padding row reads the last real row and is zeroed afterwards.
    //          The raw gate rows stay in registers for the gate VJP at the end of the tile. ----
    constexpr int NPASS = 64 / BG_PASS_ROWS;
    float gvs[NPASS][8];
    uint2 qs0[NPASS], qs1[NPASS], ks0[NPASS], ks1[NPASS];
#pragma unroll
    for (int n = 0; n < NPASS; ++n) {
        const int row = (tid >> 4) + BG_PASS_ROWS * n, lrow = min(row, ci.valid - 1);
        const size_t off = base + (size_t)lrow * tok_stride + 4 * pc;
        if (p.g_per_head) {        // one gate per (token, head), shared by all channels
            const size_t gi = (size_t)(ci.row0 + lrow) * p.H + h;
            const float gs = p.g_fp32 ? reinterpret_cast<const float*>(p.g)[gi]
                                      : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.g)[gi]);
#pragma unroll
            for (int e = 0; e < 8; ++e) gvs[n][e] = gs;
        } else if (p.g_fp32) {
            const float4 lo = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.g) + off);
            const float4 hi = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.g) + off + 64);
            gvs[n][0] = lo.x; gvs[n][1] = lo.y; gvs[n][2] = lo.z; gvs[n][3] = lo.w;
            gvs[n][4] = hi.x; gvs[n][5] = hi.y; gvs[n][6] = hi.z; gvs[n][7] = hi.w;
        } else {
            const uint2 lo = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.g) + off);
            const uint2 hi = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.g) + off + 64);
            // kept as packed bits until used: nothing depends on the loads yet
            gvs[n][0] = __uint_as_float(lo.x); gvs[n][1] = __uint_as_float(lo.y);
            gvs[n][2] = __uint_as_float(hi.x); gvs[n][3] = __uint_as_float(hi.y);
        }
        qs0[n] = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.q) + off);
        qs1[n] = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.q) + off + 64);
        ks0[n] = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.k) + off);
        ks1[n] = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.k) + off + 64);
    }
    // the other per-tile inputs of this phase, fetched now as raw bits: beta, the beta-gradient partial of the dense
    // stage, and (I + L)^-1
    uint32_t beta_bits = 0;
    float dbu_pre = 0.f;
    if (tid < 64) {
        const size_t bi = (size_t)(ci.row0 + min(tid, ci.valid - 1)) * p.H + h;
        beta_bits = p.beta_fp32 ? reinterpret_cast<const uint32_t*>(p.beta)[bi] : (uint32_t)reinterpret_cast<const uint16_t*>(p.beta)[bi];
        dbu_pre = scr[SCR_DBU + tid];
    }
    float4 a_pre[64 * 16 / BG_THREADS];
#pragma unroll
    for (int n = 0; n < 64 * 16 / BG_THREADS; ++n) {
        const int i = tid + BG_THREADS * n;
        a_pre[n] = *reinterpret_cast<const float4*>(p.akk + tile_idx * 4096 + (i >> 4) * 64 + (i & 15) * 4);
    }
    const bool g_packed = !p.g_per_head && !p.g_fp32;       // gvs[n][0..3] hold 8 bf16 values
    auto gate_row = [&](int n, float (&gv)[8]) {
        if (g_packed) {
            float2 f;
            f = unpack_bf16(__float_as_uint(gvs[n][0])); gv[0] = f.x; gv[1] = f.y;
            f = unpack_bf16(__float_as_uint(gvs[n][1])); gv[2] = f.x; gv[3] = f.y;
            f = unpack_bf16(__float_as_uint(gvs[n][2])); gv[4] = f.x; gv[5] = f.y;
            f = unpack_bf16(__float_as_uint(gvs[n][3])); gv[6] = f.x; gv[7] = f.y;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) gv[e] = gvs[n][e];
        }
    };
#pragma unroll
    for (int n = 0; n < NPASS; ++n) {
        const int row = (tid >> 4) + BG_PASS_ROWS * n;
        const bool live = row < ci.valid;
        float gv[8];
        gate_row(n, gv);
        const uint2 zero2 = make_uint2(0, 0);
        const uint2 q0 = live ? qs0[n] : zero2, q1 = live ? qs1[n] : zero2, k0 = live ? ks0[n] : zero2, k1 = live ? ks1[n] : zero2;
        float a[8];
#pragma unroll
        for (int e = 0; e < 8; ++e)
            a[e] = live ? RCP_LN2 * bg_gate(gv[e], bias[e], alpha, p.gate_mode, p.lower_bound) : 0.f;
        *reinterpret_cast<float4*>(sG + row * GS + 4 * pc) = make_float4(a[0], a[1], a[2], a[3]);
        *reinterpret_cast<float4*>(sG + row * GS + 64 + 4 * pc) = make_float4(a[4], a[5], a[6], a[7]);
        *reinterpret_cast<uint2*>(sQ + row * QS + 4 * pc) = q0;
        *reinterpret_cast<uint2*>(sQ + row * QS + 64 + 4 * pc) = q1;
        *reinterpret_cast<uint2*>(sK + row * QS + 4 * pc) = k0;
        *reinterpret_cast<uint2*>(sK + row * QS + 64 + 4 * pc) = k1;
        float sq = 0.f, sk = 0.f;
        {
            const uint32_t qw[4] = {q0.x, q0.y, q1.x, q1.y}, kw[4] = {k0.x, k0.y, k1.x, k1.y};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float2 f = unpack_bf16(qw[e]);
                sq += f.x * f.x + f.y * f.y;
                f = unpack_bf16(kw[e]);
                sk += f.x * f.x + f.y * f.y;
            }
        }
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) {
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
            sk += __shfl_xor_sync(0xffffffffu, sk, o);
        }
        if (pc == 0) {
            rstd_q[row] = p.use_l2norm ? rsqrtf(sq + 1e-6f) : 1.f;
            rstd_k[row] = p.use_l2norm ? rsqrtf(sk + 1e-6f) : 1.f;
        }
    }
    if (tid < 64) {
        float b = 0.f;
        if (tid < ci.valid) {
            b = p.beta_fp32 ? __uint_as_float(beta_bits) : __uint_as_float(beta_bits << 16);
            if (p.beta_logit) b = __fdividef(1.f, 1.f + __expf(-b));
        }
        sBeta[tid] = b;
        sDbeta[tid] = dbu_pre;
    }
    if (tid < 128) sCol[tid] = 0.f;
#pragma unroll
    for (int n = 0; n < 64 * 16 / BG_THREADS; ++n) {
        const int i = tid + BG_THREADS * n, row = i >> 4, c4 = (i & 15) * 4;
        const float4 a = a_pre[n];
        *reinterpret_cast<float4*>(sA + row * AR + c4) = make_float4(bg_tf32(a.x), bg_tf32(a.y), bg_tf32(a.z), bg_tf32(a.w));
    }
    __syncthreads();
    BG_MARK(0);   // loads, gate, norms
    // ---- 1b. cumulative sum down the rows (a row segment per thread, then the earlier segments' totals are added) ----
    {
        const int d = tid & 127, seg = tid >> 7;
        float run = 0.f;
#pragma unroll 8
        for (int r = 0; r < BG_SEG_ROWS; ++r) {
            const int row = seg * BG_SEG_ROWS + r;
            run += sG[row * GS + d];
            sG[row * GS + d] = run;
        }
        sHalf[seg * 128 + d] = run;
        __syncthreads();
        float t0 = 0.f;
        for (int s2 = 0; s2 < seg; ++s2) t0 += sHalf[s2 * 128 + d];
        if (seg > 0) {
#pragma unroll 8
            for (int r = 0; r < BG_SEG_ROWS; ++r) sG[(seg * BG_SEG_ROWS + r) * GS + d] += t0;
        }
    }
    __syncthreads();

    BG_MARK(1);   // cumulative sum
    // ---- 2. stage dW (acc1) and X = beta k-hat 2^G (acc3), both rounded to tf32 (unrolled: loads in flight together) ----
#pragma unroll
    for (int i = tid; i < 64 * 32; i += BG_THREADS) {
        const int row = i >> 5, c4 = (i & 31) * 4;
        const float4 w = *reinterpret_cast<const float4*>(scr + SCR_DW + row * DK + c4);
        *reinterpret_cast<float4*>(acc1 + row * AS + c4) = make_float4(bg_tf32(w.x), bg_tf32(w.y), bg_tf32(w.z), bg_tf32(w.w));
        const float bk = sBeta[row] * rstd_k[row];
        float x[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
            x[e] = bg_tf32(bk * __bfloat162float(sK[row * QS + c4 + e]) * fast_exp2(sG[row * GS + c4 + e]));
        *reinterpret_cast<float4*>(acc3 + row * AS + c4) = make_float4(x[0], x[1], x[2], x[3]);
    }
    __syncthreads();

    BG_MARK(2);   // stage dW, X
    const int mt = warp & 3, nh = warp >> 2;     // 16-row tile and column group of this warp in the GEMM phases
    const int r0 = 16 * mt + g8, r1 = r0 + 8;
    // Fragments that are read the way they are stored (A: row = token, K contiguous; B: row = n, K contiguous) come from
    // ldmatrix: an 8 x 8 b16 tile is an 8 x 4 tile of 32-bit words and lane l receives word (row l / 4, column l % 4),
    // which is the m16n8k8 tf32 fragment layout -- one x4 load is a whole A fragment or the B fragments of two n-tiles
    // instead of four scalar shared-memory loads each (the LSU is this kernel's busiest pipe).
    const uint32_t sm_u32 = smem_u32(sm);
    const int lr = lane & 7, lm = lane >> 3;
    auto ldsm_a = [&](int base_floats, int stride, int row0, int k0, float (&f)[4]) {
        ldsm_x4(sm_u32 + (uint32_t)((base_floats + (row0 + lr + 8 * (lm & 1)) * stride + k0 + 4 * (lm >> 1)) * 4),
                reinterpret_cast<uint32_t&>(f[0]), reinterpret_cast<uint32_t&>(f[1]), reinterpret_cast<uint32_t&>(f[2]),
                reinterpret_cast<uint32_t&>(f[3]));
    };
    auto ldsm_b2 = [&](int base_floats, int stride, int n0, int k0, float (&f)[4]) {     // f[0..1]: n-tile n0, f[2..3]: n-tile n0 + 8
        ldsm_x4(sm_u32 + (uint32_t)((base_floats + (n0 + lr + 8 * (lm >> 1)) * stride + k0 + 4 * (lm & 1)) * 4),
                reinterpret_cast<uint32_t&>(f[0]), reinterpret_cast<uint32_t&>(f[1]), reinterpret_cast<uint32_t&>(f[2]),
                reinterpret_cast<uint32_t&>(f[3]));
    };

    // ---- 3. dA = dAu + stril(dW X^T) -> c2 (zero on and above the diagonal) ----
    {
        float acc[BG_NT64][4];
#pragma unroll
        for (int nt = 0; nt < BG_NT64; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        if (8 * BG_NT64 * nh <= 16 * mt + 15) {
#pragma unroll 4
            for (int ks = 0; ks < 16; ++ks) {
                const int k0 = 8 * ks;
                float fa[4], fb[4];
                ldsm_a(BG_ACC1, AS, 16 * mt, k0, fa);
                static_assert(BG_NT64 == 2, "one x4 load covers the B fragments of the warp's two n-tiles");
                ldsm_b2(BG_ACC3, AS, 8 * BG_NT64 * nh, k0, fb);
                bg_mma(acc[0], fa, fb[0], fb[1]);
                bg_mma(acc[1], fa, fb[2], fb[3]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < BG_NT64; ++nt) {
            const int col = 8 * BG_NT64 * nh + 8 * nt + 2 * t4;
            const float2 u0 = *reinterpret_cast<const float2*>(scr + SCR_DAU + r0 * BT + col);
            const float2 u1 = *reinterpret_cast<const float2*>(scr + SCR_DAU + r1 * BT + col);
            c2[r0 * AR + col] = (col < r0) ? bg_tf32(acc[nt][0] + u0.x) : 0.f;
            c2[r0 * AR + col + 1] = (col + 1 < r0) ? bg_tf32(acc[nt][1] + u0.y) : 0.f;
            c2[r1 * AR + col] = (col < r1) ? bg_tf32(acc[nt][2] + u1.x) : 0.f;
            c2[r1 * AR + col + 1] = (col + 1 < r1) ? bg_tf32(acc[nt][3] + u1.y) : 0.f;
        }
    }
    __syncthreads();
    BG_MARK(3);   // dA
    // ---- 4a. T1 = dA A^T -> c1 ----
    {
        float acc[BG_NT64][4];
#pragma unroll
        for (int nt = 0; nt < BG_NT64; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        for (int ks = 0; ks < 2 * mt + 2; ++ks) {          // dA[i][j] = 0 for j >= i: later k-steps contribute nothing
            const int k0 = 8 * ks;
            float fa[4], fb[4];
            ldsm_a(BG_C2, AR, 16 * mt, k0, fa);
            ldsm_b2(BG_A, AR, 8 * BG_NT64 * nh, k0, fb);
            bg_mma(acc[0], fa, fb[0], fb[1]);
            bg_mma(acc[1], fa, fb[2], fb[3]);
        }
#pragma unroll
        for (int nt = 0; nt < BG_NT64; ++nt) {
            const int col = 8 * BG_NT64 * nh + 8 * nt + 2 * t4;
            c1[r0 * AR + col] = bg_tf32(acc[nt][0]);
            c1[r0 * AR + col + 1] = bg_tf32(acc[nt][1]);
            c1[r1 * AR + col] = bg_tf32(acc[nt][2]);
            c1[r1 * AR + col + 1] = bg_tf32(acc[nt][3]);
        }
    }
    __syncthreads();
    // ---- 4b. dL = -stril(A^T T1); dbeta += rowsum(dL * M); cR = beta_i dL -> c2 ----
    {
        float acc[BG_NT64][4];
#pragma unroll
        for (int nt = 0; nt < BG_NT64; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        for (int ks = 2 * mt; ks < 8; ++ks) {              // A[m][i] = 0 for m < i
            const int k0 = 8 * ks;
            const float fa[4] = {sA[(k0 + t4) * AR + r0], sA[(k0 + t4) * AR + r1], sA[(k0 + t4 + 4) * AR + r0], sA[(k0 + t4 + 4) * AR + r1]};
#pragma unroll
            for (int nt = 0; nt < BG_NT64; ++nt) {
                const int j = 8 * BG_NT64 * nh + 8 * nt + g8;
                bg_mma(acc[nt], fa, c1[(k0 + t4) * AR + j], c1[(k0 + t4 + 4) * AR + j]);
            }
        }
        const float b0 = sBeta[r0], b1 = sBeta[r1];
        const float* mk = p.mkk + tile_idx * 4096;
        float db0 = 0.f, db1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < BG_NT64; ++nt) {
            const int col = 8 * BG_NT64 * nh + 8 * nt + 2 * t4;
            const float2 m0 = *reinterpret_cast<const float2*>(mk + r0 * BT + col);
            const float2 m1 = *reinterpret_cast<const float2*>(mk + r1 * BT + col);
            const float v00 = (col < r0) ? -acc[nt][0] : 0.f, v01 = (col + 1 < r0) ? -acc[nt][1] : 0.f;
            const float v10 = (col < r1) ? -acc[nt][2] : 0.f, v11 = (col + 1 < r1) ? -acc[nt][3] : 0.f;
            db0 += v00 * m0.x + v01 * m0.y;
            db1 += v10 * m1.x + v11 * m1.y;
            c2[r0 * AR + col] = bg_tf32(b0 * v00);
            c2[r0 * AR + col + 1] = bg_tf32(b0 * v01);
            c2[r1 * AR + col] = bg_tf32(b1 * v10);
            c2[r1 * AR + col + 1] = bg_tf32(b1 * v11);
        }
        db0 += __shfl_xor_sync(0xffffffffu, db0, 1); db0 += __shfl_xor_sync(0xffffffffu, db0, 2);
        db1 += __shfl_xor_sync(0xffffffffu, db1, 1); db1 += __shfl_xor_sync(0xffffffffu, db1, 2);
        if (t4 == 0) {
            pBeta[nh * 64 + r0] = db0;
            pBeta[nh * 64 + r1] = db1;
        }
    }
    __syncthreads();
    BG_MARK(4);   // T1, dL
    if (tid < 64) {
        float v = 0.f;
#pragma unroll
        for (int x = 0; x < BG_NQ; ++x) v += pBeta[x * 64 + tid];
        sDbeta[tid] += v;
    }
#pragma unroll
    for (int x = tid; x < 64 * 16; x += BG_THREADS) {      // cP = scale * dPs -> c1 (T1 is no longer needed)
        const int row = x >> 4, c4 = (x & 15) * 4;
        const float4 v = *reinterpret_cast<const float4*>(scr + SCR_DPS + row * BT + c4);
        *reinterpret_cast<float4*>(c1 + row * AR + c4) =
            make_float4(bg_tf32(p.scale * v.x), bg_tf32(p.scale * v.y), bg_tf32(p.scale * v.z), bg_tf32(p.scale * v.w));
    }

    // ---- 5. Zw = A^T dW (gradient w.r.t. X); initial values of the dq-hat, dk-hat and dG accumulators ----
    {
        float zw[BG_NT128][4];
#pragma unroll
        for (int nt = 0; nt < BG_NT128; ++nt) zw[nt][0] = zw[nt][1] = zw[nt][2] = zw[nt][3] = 0.f;
        // the scratch-record entries this thread combines with Zw below: fetched now, so that the loads run under the MMAs
        float2 dqg_pre[BG_NT128][2], dkg_pre[BG_NT128][2];
#pragma unroll
        for (int nt = 0; nt < BG_NT128; ++nt) {
            const int col = 8 * BG_NT128 * nh + 8 * nt + 2 * t4;
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int row = rr ? r1 : r0;
                dqg_pre[nt][rr] = *reinterpret_cast<const float2*>(scr + SCR_DQG + row * DK + col);
                dkg_pre[nt][rr] = *reinterpret_cast<const float2*>(scr + SCR_DKG + row * DK + col);
            }
        }
        for (int ks = 2 * mt; ks < 8; ++ks) {
            const int k0 = 8 * ks;
            const float fa[4] = {sA[(k0 + t4) * AR + r0], sA[(k0 + t4) * AR + r1], sA[(k0 + t4 + 4) * AR + r0], sA[(k0 + t4 + 4) * AR + r1]};
#pragma unroll
            for (int nt = 0; nt < BG_NT128; ++nt) {
                const int d = 8 * BG_NT128 * nh + 8 * nt + g8;
                bg_mma(zw[nt], fa, acc1[(k0 + t4) * AS + d], acc1[(k0 + t4 + 4) * AS + d]);
            }
        }
        __syncthreads();                                   // every warp has finished reading dW from acc1
        const float bb[2] = {sBeta[r0], sBeta[r1]};
        const float rq[2] = {rstd_q[r0], rstd_q[r1]}, rk[2] = {rstd_k[r0], rstd_k[r1]};
        float dbw[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < BG_NT128; ++nt) {
            const int col = 8 * BG_NT128 * nh + 8 * nt + 2 * t4;
            const float2 gl = *reinterpret_cast<const float2*>(sG + 63 * GS + col);
            float cs0 = 0.f, cs1 = 0.f;                    // column sums of dKg * Kg over this thread's two rows
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int row = rr ? r1 : r0;
                const float2 gi = *reinterpret_cast<const float2*>(sG + row * GS + col);
                const float2 dqg = dqg_pre[nt][rr], dkg = dkg_pre[nt][rr];
                const float2 qf = unpack_bf16(*reinterpret_cast<const uint32_t*>(sQ + row * QS + col));
                const float2 kf = unpack_bf16(*reinterpret_cast<const uint32_t*>(sK + row * QS + col));
                const float gg[2] = {gi.x, gi.y}, gls[2] = {gl.x, gl.y}, dq2[2] = {dqg.x, dqg.y}, dk2[2] = {dkg.x, dkg.y};
                const float qh[2] = {qf.x * rq[rr], qf.y * rq[rr]}, kh[2] = {kf.x * rk[rr], kf.y * rk[rr]};
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float z = zw[nt][2 * rr + e];
                    const float eg = fast_exp2(gg[e]), ekg = fast_exp2(gls[e] - gg[e]);
                    const float dkp = bb[rr] * z, kplus = kh[e] * eg, kgv = kh[e] * ekg, qgv = p.scale * qh[e] * eg;
                    acc1[row * AS + col + e] = p.scale * dq2[e] * eg;
                    acc2[row * AS + col + e] = dkp * eg + dk2[e] * ekg;
                    acc3[row * AS + col + e] = dq2[e] * qgv + dkp * kplus - dk2[e] * kgv;
                    dbw[rr] = fmaf(z, kplus, dbw[rr]);
                    if (e == 0) cs0 = fmaf(dk2[e], kgv, cs0); else cs1 = fmaf(dk2[e], kgv, cs1);
                }
            }
            // sum over the 8 row pairs of this warp (lanes with equal t4): columns col, col+1
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                cs0 += __shfl_xor_sync(0xffffffffu, cs0, o);
                cs1 += __shfl_xor_sync(0xffffffffu, cs1, o);
            }
            if (g8 == 0) {
                pGl[mt * 128 + col] = cs0;
                pGl[mt * 128 + col + 1] = cs1;
            }
        }
        dbw[0] += __shfl_xor_sync(0xffffffffu, dbw[0], 1); dbw[0] += __shfl_xor_sync(0xffffffffu, dbw[0], 2);
        dbw[1] += __shfl_xor_sync(0xffffffffu, dbw[1], 1); dbw[1] += __shfl_xor_sync(0xffffffffu, dbw[1], 2);
        if (t4 == 0) {
            pBeta[nh * 64 + r0] = dbw[0];
            pBeta[nh * 64 + r1] = dbw[1];
        }
    }
    __syncthreads();
    if (tid < 64) {
        float v = 0.f;
#pragma unroll
        for (int x = 0; x < BG_NQ; ++x) v += pBeta[x * 64 + tid];
        sDbeta[tid] += v;
    }
    if (tid < 128) {   // g_last sits in row 63 (padding rows repeat the last real value): fold its gradient in there
        const float dgl = (pGl[tid] + pGl[128 + tid]) + (pGl[256 + tid] + pGl[384 + tid]) +
                          fast_exp2(sG[63 * GS + tid]) * scr[SCR_DD + tid];
        acc3[63 * AS + tid] += dgl;
    }
    __syncthreads();

    BG_MARK(5);   // Zw, accumulator initial values
    // ---- next tile of this CTA: pull its inputs into L2 while the Gram phase computes (the first tile comes cold).
    //      Bulk prefetches: one instruction covers a whole contiguous array or a whole token row ----
    if (next_tile >= 0) {
        if (tid == 0) {
            bulk_prefetch_l2(p.scratch + (size_t)next_tile * (size_t)BWD_SCRATCH_FLOATS, BWD_SCRATCH_FLOATS * 4);
            bulk_prefetch_l2(p.akk + (size_t)next_tile * 4096, 4096 * 4);
            bulk_prefetch_l2(p.mkk + (size_t)next_tile * 4096, 4096 * 4);
        } else if (tid >= 32 && tid < 32 + 64 * 3) {
            const int cn = next_tile / p.H, hn = next_tile - cn * p.H;
            const ChunkInfo cin = chunk_info(cn, p.cu_seqlens, p.chunk_indices, p.T);
            const int row = (tid - 32) & 63, which = (tid - 32) >> 6;      // q, k, g
            if (row < cin.valid) {
                const size_t o = (size_t)(cin.row0 + row) * tok_stride + (size_t)hn * DK;
                if (which < 2) bulk_prefetch_l2(reinterpret_cast<const __nv_bfloat16*>(which ? p.k : p.q) + o, DK * 2);
                else if (p.g_per_head) { /* a few bytes per row: no hint */ }
                else if (p.g_fp32) bulk_prefetch_l2(reinterpret_cast<const float*>(p.g) + o, DK * 4);
                else bulk_prefetch_l2(reinterpret_cast<const __nv_bfloat16*>(p.g) + o, DK * 2);
            }
        }
    }

    BG_MARK(6);   // L2 hints
    // ---- 6. VJPs of the gated Gram matrices. Warp w owns 128 / BG_WARPS key channels for all 64 rows; the same
    //         thread owns the same (row, channel) cells in the row-side and column-side updates: no synchronisation ----
    {
        const int dB0 = 8 * BG_NT6 * warp + g8;          // channel of this lane's B-fragment column in n-tile 0 (+8 per n-tile)
#pragma unroll 1
        for (int I = 0; I < 4; ++I) {                     // row side: rows of block I against columns j < 16(I+1)
            float accP[BG_NT6][4], accR[BG_NT6][4];
#pragma unroll
            for (int nt = 0; nt < BG_NT6; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) accP[nt][e] = accR[nt][e] = 0.f;
            const int i0 = 16 * I + g8, i1 = i0 + 8;
            float rIv[BG_NT6];
#pragma unroll
            for (int nt = 0; nt < BG_NT6; ++nt) rIv[nt] = sG[16 * I * GS + dB0 + 8 * nt];
            for (int ks = 0; ks < 2 * I + 2; ++ks) {
                const int j0 = 8 * ks + t4, j1 = j0 + 4;
                float aP[4], aR[4];
                ldsm_a(BG_C1, AR, 16 * I, 8 * ks, aP);
                ldsm_a(BG_C2, AR, 16 * I, 8 * ks, aR);
                const float k0s = rstd_k[j0], k1s = rstd_k[j1];
#pragma unroll
                for (int nt = 0; nt < BG_NT6; ++nt) {
                    const int d = dB0 + 8 * nt;
                    const float rI = rIv[nt];
                    const float b0 = __bfloat162float(sK[j0 * QS + d]) * k0s * fast_exp2(fminf(rI - sG[j0 * GS + d], 120.f));
                    const float b1 = __bfloat162float(sK[j1 * QS + d]) * k1s * fast_exp2(fminf(rI - sG[j1 * GS + d], 120.f));
                    const float h0 = bg_tf32(b0), h1 = bg_tf32(b1), l0 = bg_tf32_lo(b0 - h0), l1 = bg_tf32_lo(b1 - h1);
                    bg_mma(accP[nt], aP, l0, l1);
                    bg_mma(accP[nt], aP, h0, h1);
                    bg_mma(accR[nt], aR, l0, l1);
                    bg_mma(accR[nt], aR, h0, h1);
                }
            }
#pragma unroll
            for (int nt = 0; nt < BG_NT6; ++nt) {
                const int col = 8 * BG_NT6 * warp + 8 * nt + 2 * t4;
                const float2 rI = *reinterpret_cast<const float2*>(sG + 16 * I * GS + col);
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int row = rr ? i1 : i0;
                    const float2 gi = *reinterpret_cast<const float2*>(sG + row * GS + col);
                    const float2 qf = unpack_bf16(*reinterpret_cast<const uint32_t*>(sQ + row * QS + col));
                    const float2 kf = unpack_bf16(*reinterpret_cast<const uint32_t*>(sK + row * QS + col));
                    const float f0 = fast_exp2(gi.x - rI.x), f1 = fast_exp2(gi.y - rI.y);
                    const float dq0 = f0 * accP[nt][2 * rr], dq1 = f1 * accP[nt][2 * rr + 1];
                    const float dk0 = f0 * accR[nt][2 * rr], dk1 = f1 * accR[nt][2 * rr + 1];
                    acc1[row * AS + col] += dq0;
                    acc1[row * AS + col + 1] += dq1;
                    acc2[row * AS + col] += dk0;
                    acc2[row * AS + col + 1] += dk1;
                    acc3[row * AS + col] += rstd_q[row] * qf.x * dq0 + rstd_k[row] * kf.x * dk0;
                    acc3[row * AS + col + 1] += rstd_q[row] * qf.y * dq1 + rstd_k[row] * kf.y * dk1;
                }
            }
        }
        BG_MARK(7);   // Gram VJP, row side
#pragma unroll 1
        for (int J = 0; J < 4; ++J) {                     // column side: columns of block J against rows i >= 16J
            float accC[BG_NT6][4];
#pragma unroll
            for (int nt = 0; nt < BG_NT6; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) accC[nt][e] = 0.f;
            const int jc0 = 16 * J + g8, jc1 = jc0 + 8;
            float sJv[BG_NT6];
#pragma unroll
            for (int nt = 0; nt < BG_NT6; ++nt) sJv[nt] = sG[(16 * J + 15) * GS + dB0 + 8 * nt];
            for (int ks = 2 * J; ks < 8; ++ks) {
                const int ia = 8 * ks + t4, ib = ia + 4;
                const float aP[4] = {c1[ia * AR + jc0], c1[ia * AR + jc1], c1[ib * AR + jc0], c1[ib * AR + jc1]};
                const float aR[4] = {c2[ia * AR + jc0], c2[ia * AR + jc1], c2[ib * AR + jc0], c2[ib * AR + jc1]};
                const float qa = rstd_q[ia], qb = rstd_q[ib], ka = rstd_k[ia], kb = rstd_k[ib];
#pragma unroll
                for (int nt = 0; nt < BG_NT6; ++nt) {
                    const int d = dB0 + 8 * nt;
                    const float sJ = sJv[nt];
                    const float ea = fast_exp2(fminf(sG[ia * GS + d] - sJ, 120.f)), eb = fast_exp2(fminf(sG[ib * GS + d] - sJ, 120.f));
                    bg_mma_split(accC[nt], aP, __bfloat162float(sQ[ia * QS + d]) * qa * ea, __bfloat162float(sQ[ib * QS + d]) * qb * eb);
                    bg_mma_split(accC[nt], aR, __bfloat162float(sK[ia * QS + d]) * ka * ea, __bfloat162float(sK[ib * QS + d]) * kb * eb);
                }
            }
#pragma unroll
            for (int nt = 0; nt < BG_NT6; ++nt) {
                const int col = 8 * BG_NT6 * warp + 8 * nt + 2 * t4;
                const float2 sJ = *reinterpret_cast<const float2*>(sG + (16 * J + 15) * GS + col);
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int row = rr ? jc1 : jc0;
                    const float2 gj = *reinterpret_cast<const float2*>(sG + row * GS + col);
                    const float2 kf = unpack_bf16(*reinterpret_cast<const uint32_t*>(sK + row * QS + col));
                    const float d0 = fast_exp2(sJ.x - gj.x) * accC[nt][2 * rr], d1 = fast_exp2(sJ.y - gj.y) * accC[nt][2 * rr + 1];
                    acc2[row * AS + col] += d0;
                    acc2[row * AS + col + 1] += d1;
                    acc3[row * AS + col] -= rstd_k[row] * kf.x * d0;
                    acc3[row * AS + col + 1] -= rstd_k[row] * kf.y * d1;
                }
            }
        }
    }
    __syncthreads();
    BG_MARK(8);   // Gram VJP, column side

    // ---- 7a. reverse cumulative sum of dG down the rows, in place (a row segment per thread, then the later segments' totals) ----
    {
        const int d = tid & 127, seg = tid >> 7;
        float run = 0.f;
#pragma unroll 8
        for (int r = BG_SEG_ROWS - 1; r >= 0; --r) {
            const int row = seg * BG_SEG_ROWS + r;
            run += acc3[row * AS + d];
            acc3[row * AS + d] = run;
        }
        sHalf[seg * 128 + d] = run;
        __syncthreads();
        float t1 = 0.f;
        for (int s2 = BG_SEG - 1; s2 > seg; --s2) t1 += sHalf[s2 * 128 + d];
        if (seg < BG_SEG - 1) {
#pragma unroll 8
            for (int r = 0; r < BG_SEG_ROWS; ++r) acc3[(seg * BG_SEG_ROWS + r) * AS + d] += t1;
        }
    }
    __syncthreads();
    BG_MARK(9);   // reverse cumulative sum
    // ---- 7b. gate VJP with wide accesses: dg, per-channel sums for d dt_bias, the A_log sum ----
    float dA_part = 0.f;
    {
        float colsum[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) colsum[e] = 0.f;
#pragma unroll
        for (int n = 0; n < 64 / BG_PASS_ROWS; ++n) {
            const int row = (tid >> 4) + BG_PASS_ROWS * n;
            if (row >= ci.valid) continue;       // uniform over the 16 lanes that share a row
            const size_t off = base + (size_t)row * tok_stride + 4 * pc;
            float gv[8], dx[8];
            gate_row(n, gv);             // the raw gate values loaded at the top of the tile
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int d = 64 * (e >> 2) + 4 * pc + (e & 3);
                const float da = acc3[row * AS + d] * gs_inv;       // gradient w.r.t. the natural-log decay a_row[d]
                float v = da;
                if (p.gate_mode == GATE_LOWER_BOUND) {
                    const float x = gv[e] + bias[e];
                    const float sg = fast_rcp(1.f + fast_exp2(-alpha * RCP_LN2 * x));
                    v = da * p.lower_bound * sg * (1.f - sg) * alpha;
                    dA_part = fmaf(v, x, dA_part);
                    colsum[e] += v;
                } else if (p.gate_mode == GATE_SOFTPLUS) {
                    const float x = gv[e] + bias[e];
                    const float sg = __fdividef(1.f, 1.f + __expf(-x));
                    const float sp = x > 20.f ? x : log1pf(__expf(x));
                    v = -da * alpha * sg;
                    dA_part = fmaf(da, -alpha * sp, dA_part);
                    colsum[e] += v;
                }
                dx[e] = v;
            }
            if (p.g_per_head) {        // the gate is shared by the 128 channels: its gradient is their sum
                float sum = ((dx[0] + dx[1]) + (dx[2] + dx[3])) + ((dx[4] + dx[5]) + (dx[6] + dx[7]));
                const unsigned half_mask = lane < 16 ? 0x0000ffffu : 0xffff0000u;     // the other half may hold a padding row
#pragma unroll
                for (int o = 1; o < 16; o <<= 1) sum += __shfl_xor_sync(half_mask, sum, o);
                if (pc == 0) {
                    const size_t gi = (size_t)(ci.row0 + row) * p.H + h;
                    if (p.g_fp32) reinterpret_cast<float*>(p.dg)[gi] = sum;
                    else reinterpret_cast<__nv_bfloat16*>(p.dg)[gi] = __float2bfloat16_rn(sum);
                }
            } else if (p.g_fp32) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.dg) + off) = make_float4(dx[0], dx[1], dx[2], dx[3]);
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.dg) + off + 64) = make_float4(dx[4], dx[5], dx[6], dx[7]);
            } else {
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.dg) + off) =
                    make_uint2(pack_bf16(dx[0], dx[1]), pack_bf16(dx[2], dx[3]));
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.dg) + off + 64) =
                    make_uint2(pack_bf16(dx[4], dx[5]), pack_bf16(dx[6], dx[7]));
            }
        }
        if (p.gate_mode != GATE_NONE && p.ddt_bias) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                // lanes l and l+16 hold the same channels: combine them, then one shared-memory atomic per channel and warp
                float v = colsum[e] + __shfl_xor_sync(0xffffffffu, colsum[e], 16);
                if (lane < 16) atomicAdd(&sCol[64 * (e >> 2) + 4 * pc + (e & 3)], v);
            }
        }
    }
    if (p.gate_mode != GATE_NONE && p.dA_log) {
#pragma unroll
        for (int o = 16; o; o >>= 1) dA_part += __shfl_xor_sync(0xffffffffu, dA_part, o);
        if (lane == 0) sRed[warp] = dA_part;
    }
    __syncthreads();
    if (p.gate_mode != GATE_NONE) {
        if (p.ddt_bias && tid < 128) atomicAdd(&p.ddt_bias[h * DK + tid], sCol[tid]);
        if (p.dA_log && tid == 0) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < BG_WARPS; ++w) v += sRed[w];
            atomicAdd(&p.dA_log[h], v);
        }
    }

    BG_MARK(10);  // gate VJP, dg
    // ---- 8. L2-norm VJP and stores of dq, dk (a warp per row); dbeta ----
    for (int r = 0; r < 64 / BG_WARPS; ++r) {
        const int row = warp * (64 / BG_WARPS) + r;
        if (row >= ci.valid) continue;
        float dq[4], dk[4], qh[4], kh[4];
        float sq = 0.f, sk = 0.f;
        const float4 a1 = *reinterpret_cast<const float4*>(acc1 + row * AS + lane * 4);
        const float4 a2 = *reinterpret_cast<const float4*>(acc2 + row * AS + lane * 4);
        const uint2 qr = *reinterpret_cast<const uint2*>(sQ + row * QS + lane * 4);
        const uint2 kr = *reinterpret_cast<const uint2*>(sK + row * QS + lane * 4);
        dq[0] = a1.x * gs_inv; dq[1] = a1.y * gs_inv; dq[2] = a1.z * gs_inv; dq[3] = a1.w * gs_inv;
        dk[0] = a2.x * gs_inv; dk[1] = a2.y * gs_inv; dk[2] = a2.z * gs_inv; dk[3] = a2.w * gs_inv;
        float2 f;
        f = unpack_bf16(qr.x); qh[0] = f.x * rstd_q[row]; qh[1] = f.y * rstd_q[row];
        f = unpack_bf16(qr.y); qh[2] = f.x * rstd_q[row]; qh[3] = f.y * rstd_q[row];
        f = unpack_bf16(kr.x); kh[0] = f.x * rstd_k[row]; kh[1] = f.y * rstd_k[row];
        f = unpack_bf16(kr.y); kh[2] = f.x * rstd_k[row]; kh[3] = f.y * rstd_k[row];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            sq = fmaf(dq[e], qh[e], sq);
            sk = fmaf(dk[e], kh[e], sk);
        }
        if (p.use_l2norm) {
#pragma unroll
            for (int o = 16; o; o >>= 1) {
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                dq[e] = rstd_q[row] * (dq[e] - qh[e] * sq);
                dk[e] = rstd_k[row] * (dk[e] - kh[e] * sk);
            }
        }
        const size_t off = base + (size_t)row * tok_stride + lane * 4;
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.dq) + off) = make_uint2(pack_bf16(dq[0], dq[1]), pack_bf16(dq[2], dq[3]));
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.dk) + off) = make_uint2(pack_bf16(dk[0], dk[1]), pack_bf16(dk[2], dk[3]));
    }
    if (tid < ci.valid) {
        const size_t bi = (size_t)(ci.row0 + tid) * p.H + h;
        float v = sDbeta[tid] * gs_inv;
        if (p.beta_logit) v *= sBeta[tid] * (1.f - sBeta[tid]);       // chain rule through the in-kernel sigmoid
        if (p.beta_fp32) reinterpret_cast<float*>(p.dbeta)[bi] = v;
        else reinterpret_cast<__nv_bfloat16*>(p.dbeta)[bi] = __float2bfloat16_rn(v);
    }
    BG_MARK(11);  // L2-norm VJP, dq, dk, dbeta
}

// Persistent: CTA b handles tiles b, b + gridDim.x, ... so that the next tile's inputs can be prefetched.
__global__ void __launch_bounds__(BG_THREADS, 1) kda_bwd_gated_kernel(const BwdGatedParams p, const int num_tiles) {
    extern __shared__ __align__(16) float sm[];
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int next = tile + gridDim.x;
        bg_tile(p, sm, tile, next < num_tiles ? next : -1);
        __syncthreads();                                  // shared memory is reused by the next tile
    }
}

}  // namespace kda

#ifdef KDA_PHASE_TIMERS
extern "C" int kda_bwd_gated_read_timers(unsigned long long* out, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out, kda_bwd_gated_timers, sizeof(kda_bwd_gated_timers));
    if (e == cudaSuccess && reset) {
        unsigned long long z[16] = {};
        e = cudaMemcpyToSymbol(kda_bwd_gated_timers, z, sizeof(z));
    }
    return (int)e;
}
#endif

extern "C" int kda_launch_bwd_gated(const kda::BwdGatedParams* p, int num_chunks, cudaStream_t stream) {
    using namespace kda;
    static_assert(BG_SMEM <= 227 * 1024, "shared memory budget");
    if (num_chunks <= 0) return 0;
    cudaError_t e = cudaFuncSetAttribute(kda_bwd_gated_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BG_SMEM);
    if (e != cudaSuccess) return (int)e;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = num_chunks * p->H;
    kda_bwd_gated_kernel<<<tiles < sms ? tiles : sms, BG_THREADS, BG_SMEM, stream>>>(*p, tiles);
    return (int)cudaGetLastError();
}
