// Chunk-parallel forward stage on tcgen05 tensor cores: one CTA per (chunk, head) fuses
//   gate activation + per-chunk cumulative sum (log2 domain), q/k L2 normalisation,
//   the gated 64x64 Gram matrices Aqk / L (one M=128 x N=160 TF32 UMMA chain, accumulators in TMEM),
//   Akk = (I + L)^-1 (blocked 16 -> 32 -> 64 inverse in fp32),
//   [w | u] = Akk [beta k 2^g | beta v] (one M=128 x N=256 FP16 UMMA chain),
//   kg = k 2^(g_last - g), qg = scale q 2^g,
// and writes the tile pack the state scan consumes (layout in kda_common.cuh).
//
// It replaces, in one launch, what the reference does with l2norm_fwd x2 (cula/kda/chunk.py:58-60),
// kda_gate_chunk_cumsum (cula/kda/chunk_fwd.py:69-78), chunk_kda_fwd_intra_cuda and
// recompute_w_u_cuda (csrc/api/kda_sm100.cu:22-120), so the fp32 gate, q-hat and k-hat never
// travel through HBM.
//
// Exponent handling ("safe gate"): 2^(g_i - g_j) is never formed directly inside an MMA operand. Row i of
// 16-row block I is scaled by 2^(g_i - r_I) (<= 1, r_I = g at the first row of the block) and column j by
// 2^(r_I - g_j), which is <= 1 for earlier blocks and at most 2^(15*5*log2 e) ~ 2^108 inside block I.
// So the B operand holds one copy of k-hat per anchor: 16 + 32 + 48 + 64 = 160 rows; the A operand
// is [q-hat ; k-hat] scaled by their own block anchors (128 rows). Column block I of the 128 x 160
// product is valid on the rows of block I only; the epilogue reads exactly those.
//
// Two CTAs are resident per SM (107 KB shared memory, 256 TMEM columns each), so one CTA's MUFU-heavy
// operand generation overlaps the other's MMA, inverse and epilogues.
#include "kda_common.cuh"
#include "kda_params.h"
#include "umma.cuh"

namespace kda {

constexpr int INTRA_THREADS = 256;              // 256 or 512 (the thread mappings below follow it)
constexpr int NWARPS = INTRA_THREADS / 32;
constexpr int RS = 512 / INTRA_THREADS;          // 64-row slots per thread in the (row, 8-lane) mapping
constexpr int RSTEP = INTRA_THREADS / 8;         // row distance between a thread's slots
constexpr int NIT = 1024 / INTRA_THREADS;        // (row, 16-lane) items per thread
constexpr int NPART = INTRA_THREADS / 128;       // row segments of the column scan

// shared-memory map (bytes from a 1024-aligned base)
constexpr int SM_OPA = 0;                 // A operand of one 64-channel half: [2 k-atoms][128 rows][128 B], SW128
constexpr int SM_OPB = 32768;             // B operand: [2 k-atoms][160 rows][128 B], SW128
constexpr int SM_G = 73728;               // G [64][128] fp32
constexpr int SM_MISC = 106496;           // beta[64], barriers, tmem base, segment totals of the column scan
constexpr int SM_TOTAL = 108544;
static_assert(SM_MISC + 512 + NPART * 128 * 4 <= SM_TOTAL, "segment totals must fit the misc region");
constexpr int KATOM_A = 16384, KATOM_B = 20480;
// regions reused once the Gram MMAs have completed
constexpr int SM_XS = SM_OPA;             // X = beta k 2^g, fp16 [2 mn-atoms][64 tokens][128 B], SW128 (MN-major B operand)
constexpr int SM_YS = SM_OPA + 16384;     // Y = beta v, same layout
constexpr int LROW = 68;                  // padded fp32 row of the 64x64 matrices
constexpr int SM_LF = SM_OPB;             // L fp32 [64][68]
constexpr int SM_AINV = SM_OPB + 17408;   // (I+L)^-1 fp32 [64][68]
constexpr int SM_TM = SM_OPB + 34816;     // scratch for the block products [32][36]
constexpr int TROW = 36;
constexpr int SM_AKK16 = SM_G;            // Akk fp16, stacked twice: [128][128 B], SW128 (K-major A operand)


__device__ __forceinline__ uint64_t sdesc_sw128(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return umma::make_sdesc(addr, lbo, sbo) | (2ull << 61);
}
__device__ __forceinline__ float to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}
__device__ __forceinline__ float4 tf32x4(float a, float b, float c, float d) {
    return make_float4(to_tf32(a), to_tf32(b), to_tf32(c), to_tf32(d));
}
__device__ __forceinline__ float load_gate_raw(const void* g, int g_fp32, size_t idx) {
    return g_fp32 ? reinterpret_cast<const float*>(g)[idx]
                  : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[idx]);
}
// kept out of line: it is instantiated per element group and the softplus path is long (instruction-cache footprint)
__device__ __noinline__ float gate_activation(float graw, float alpha, float bias, int gate_mode, float lower_bound) {
    if (gate_mode == GATE_NONE) return graw;
    float x = graw + bias;
    if (gate_mode == GATE_LOWER_BOUND) return __fdividef(lower_bound, 1.f + __expf(-alpha * x));
    return -alpha * (x > 20.f ? x : log1pf(__expf(x)));
}

// D(16x8) += A(16 x 8*KT) * B(8*KT x 8) with A, B fp32 in shared memory (row-major, strides lda/ldb),
// evaluated as three TF32 MMAs per k-step on the hi/lo split of both operands.
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(x - __uint_as_float(hi)));
}
__device__ __forceinline__ void mma_tf32_16x8x8(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
template <int KT>
__device__ __forceinline__ void mma_tile_3xtf32(const float* A, int lda, const float* B, int ldb, float (&acc)[4], int g, int t) {
#pragma unroll 1
    for (int ks = 0; ks < KT; ++ks) {
        const float af[4] = {A[g * lda + 8 * ks + t], A[(g + 8) * lda + 8 * ks + t], A[g * lda + 8 * ks + t + 4],
                             A[(g + 8) * lda + 8 * ks + t + 4]};
        const float bf[2] = {B[(8 * ks + t) * ldb + g], B[(8 * ks + t + 4) * ldb + g]};
        uint32_t ah[4], al[4], bh[2], bl[2];
#pragma unroll
        for (int e = 0; e < 4; ++e) split_tf32(af[e], ah[e], al[e]);
#pragma unroll
        for (int e = 0; e < 2; ++e) split_tf32(bf[e], bh[e], bl[e]);
        mma_tf32_16x8x8(acc, al, bh);
        mma_tf32_16x8x8(acc, ah, bl);
        mma_tf32_16x8x8(acc, ah, bh);
    }
}

__global__ void __launch_bounds__(INTRA_THREADS, 2) kda_fwd_intra_kernel(const IntraParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sm_u32 = smem_u32(sm);
    float* sG = reinterpret_cast<float*>(sm + SM_G);
    float* sBeta = reinterpret_cast<float*>(sm + SM_MISC);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + SM_MISC + 256);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + SM_MISC + 288);
    float* sHalf = reinterpret_cast<float*>(sm + SM_MISC + 512);      // [NPART][128] segment totals

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t tok_stride = (size_t)p.H * DK;
    const int l8 = tid & 7, rq = tid >> 3;

    if (tid == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_init(&bars[2], 1);
        fence_mbar_init();
    }
    if (warp == 0) umma::tmem_alloc(tmem_slot, 256);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    uint2 qraw[RS][4], kraw[RS][4];
    uint2 graw[NIT][2];             // bf16 gate rows of the (row, 16-lane) mapping; fp32 gates are loaded in place
    auto fetch_rows = [&](int t_id) {
        const int c2 = t_id / p.H, h2 = t_id - c2 * p.H;
        const ChunkInfo ci2 = chunk_info(c2, p.cu_seqlens, p.chunk_indices, p.T);
        const size_t base2 = (size_t)ci2.row0 * tok_stride + (size_t)h2 * DK;
        const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(p.q);
        const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(p.k);
#pragma unroll
        for (int rs = 0; rs < RS; ++rs) {
            const int row = rq + RSTEP * rs;
#pragma unroll
            for (int grp = 0; grp < 4; ++grp) {
                uint2 qv = make_uint2(0, 0), kv = make_uint2(0, 0);
                if (row < ci2.valid) {
                    size_t off = base2 + (size_t)row * tok_stride + 32 * grp + 4 * l8;
                    qv = *reinterpret_cast<const uint2*>(qp + off);
                    kv = *reinterpret_cast<const uint2*>(kp + off);
                }
                qraw[rs][grp] = qv;
                kraw[rs][grp] = kv;
            }
        }
        if (!p.g_fp32) {
#pragma unroll
            for (int n = 0; n < NIT; ++n) {
                const int row = (tid >> 4) + (INTRA_THREADS / 16) * n;
                graw[n][0] = graw[n][1] = make_uint2(0, 0);
                if (row < ci2.valid) {
                    const __nv_bfloat16* gp = reinterpret_cast<const __nv_bfloat16*>(p.g) + base2 + (size_t)row * tok_stride + 4 * (tid & 15);
                    graw[n][0] = *reinterpret_cast<const uint2*>(gp);
                    graw[n][1] = *reinterpret_cast<const uint2*>(gp + 64);
                }
            }
        }
    };
    if ((int)blockIdx.x < p.num_tiles) fetch_rows(blockIdx.x);

    // persistent over (chunk, head) tiles; the completion barriers flip phase once per tile
    for (int tile_id = blockIdx.x, iter = 0; tile_id < p.num_tiles; tile_id += gridDim.x, ++iter) {
    const uint32_t par = iter & 1;
    const int c = tile_id / p.H, h = tile_id - c * p.H;
    const ChunkInfo ci = chunk_info(c, p.cu_seqlens, p.chunk_indices, p.T);
    const size_t base = (size_t)ci.row0 * tok_stride + (size_t)h * DK;
    unsigned char* tile = p.tiles + ((size_t)c * p.H + h) * TP_BYTES;

    // q, k, g rows of this tile are already in registers: they were fetched while the previous tile was in its
    // epilogues (first tile: before the loop). Thread (rq, l8): rows rq (+RSTEP), channels 32*grp + 4*l8 .. +3.
    if (tid < 256) {   // pull this tile's v rows and the next tile's inputs towards L2 (two 128-byte lines per row)
        const int row = tid >> 2, part = tid & 3;
        if (part < 2 && row < ci.valid)
            prefetch_l2(reinterpret_cast<const __nv_bfloat16*>(p.v) + base + (size_t)row * tok_stride + 64 * part);
        const int nt = tile_id + gridDim.x;
        if (nt < p.num_tiles) {
            const int nc = nt / p.H, nh = nt - nc * p.H;
            const ChunkInfo ni = chunk_info(nc, p.cu_seqlens, p.chunk_indices, p.T);
            if (row < ni.valid) {
                const size_t nb = (size_t)(ni.row0 + row) * tok_stride + (size_t)nh * DK + 64 * (part & 1);
                if (part < 2) {
                    prefetch_l2(reinterpret_cast<const __nv_bfloat16*>(p.q) + nb);
                    prefetch_l2(reinterpret_cast<const __nv_bfloat16*>(p.k) + nb);
                } else if (p.g_fp32) {
                    prefetch_l2(reinterpret_cast<const float*>(p.g) + nb);
                    prefetch_l2(reinterpret_cast<const float*>(p.g) + nb + 32);
                } else {
                    prefetch_l2(reinterpret_cast<const __nv_bfloat16*>(p.g) + nb);
                }
            }
        }
    }

    // ---- 1a. gate activation with wide, coalesced loads: item (row, pc) covers channels 4pc..4pc+3 and
    //          64+4pc..64+4pc+3; the activated log2 decay goes to sG (zero for padding rows) ----
    {
        const float alpha = p.gate_mode != GATE_NONE ? __expf(p.A_log[h]) : 0.f;
        const int pc = tid & 15;
        float bias[8];
#pragma unroll
        for (int e = 0; e < 8; ++e)
            bias[e] = (p.gate_mode != GATE_NONE && p.dt_bias) ? p.dt_bias[h * DK + 64 * (e >> 2) + 4 * pc + (e & 3)] : 0.f;
        float gv[NIT][8];
#pragma unroll
        for (int n = 0; n < NIT; ++n) {
            const int row = (tid >> 4) + (INTRA_THREADS / 16) * n;
            const size_t off = base + (size_t)row * tok_stride + 4 * pc;
#pragma unroll
            for (int e = 0; e < 8; ++e) gv[n][e] = 0.f;
            if (row < ci.valid) {
                if (p.g_fp32) {
                    const float4 lo = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.g) + off);
                    const float4 hi = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.g) + off + 64);
                    gv[n][0] = lo.x; gv[n][1] = lo.y; gv[n][2] = lo.z; gv[n][3] = lo.w;
                    gv[n][4] = hi.x; gv[n][5] = hi.y; gv[n][6] = hi.z; gv[n][7] = hi.w;
                } else {
                    const uint2 lo = graw[n][0], hi = graw[n][1];
                    float2 f;
                    f = unpack_bf16(lo.x); gv[n][0] = f.x; gv[n][1] = f.y;
                    f = unpack_bf16(lo.y); gv[n][2] = f.x; gv[n][3] = f.y;
                    f = unpack_bf16(hi.x); gv[n][4] = f.x; gv[n][5] = f.y;
                    f = unpack_bf16(hi.y); gv[n][6] = f.x; gv[n][7] = f.y;
                }
            }
        }
#pragma unroll
        for (int n = 0; n < NIT; ++n) {
            const int row = (tid >> 4) + (INTRA_THREADS / 16) * n;
            if (p.gate_mode == GATE_LOWER_BOUND) {
                // lower_bound * sigmoid(alpha x) / ln2 with one ex2 and one rcp (flush-to-zero approximations)
                const float c0 = -alpha * RCP_LN2, c1 = (row < ci.valid) ? p.lower_bound * RCP_LN2 : 0.f;
                float a[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) a[e] = c1 * fast_rcp(1.f + fast_exp2(c0 * (gv[n][e] + bias[e])));
                *reinterpret_cast<float4*>(sG + row * DK + 4 * pc) = make_float4(a[0], a[1], a[2], a[3]);
                *reinterpret_cast<float4*>(sG + row * DK + 64 + 4 * pc) = make_float4(a[4], a[5], a[6], a[7]);
            } else {
                // other gate forms: rolled, element by element (keeps the long softplus code out of line)
                const float keep = (row < ci.valid) ? RCP_LN2 : 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    sG[row * DK + 64 * (e >> 2) + 4 * pc + (e & 3)] =
                        keep * gate_activation(gv[n][e], alpha, bias[e], p.gate_mode, p.lower_bound);
            }
        }
    }
    __syncthreads();
    // ---- 1b. cumulative sum down the rows: thread (part, d) scans its 64/NPART rows in shared memory ----
    {
        const int d = tid & 127, part = tid >> 7;
        float run = 0.f;
#pragma unroll
        for (int r = 0; r < 64 / NPART; ++r) {
            const int row = part * (64 / NPART) + r;
            run += sG[row * DK + d];
            sG[row * DK + d] = run;
        }
        sHalf[part * DK + d] = run;
    }
    // ---- 2. L2 norms from the rows held in registers, beta ----
    float rstd_q[RS], rstd_k[RS], bet[RS];
#pragma unroll
    for (int rs = 0; rs < RS; ++rs) {
        const int row = rq + RSTEP * rs;
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int grp = 0; grp < 4; ++grp) {
            float2 a = unpack_bf16(qraw[rs][grp].x), b = unpack_bf16(qraw[rs][grp].y);
            sq += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
            a = unpack_bf16(kraw[rs][grp].x); b = unpack_bf16(kraw[rs][grp].y);
            sk += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
        }
        float b = 0.f;
        if (row < ci.valid) {
            size_t bi = (size_t)(ci.row0 + row) * p.H + h;
            b = p.beta_fp32 ? reinterpret_cast<const float*>(p.beta)[bi]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.beta)[bi]);
        }
        bet[rs] = b;
        if (l8 == 0) sBeta[row] = b;
        if (p.use_l2norm) {
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
            }
            rstd_q[rs] = rsqrtf(sq + 1e-6f);
            rstd_k[rs] = rsqrtf(sk + 1e-6f);
        } else {
            rstd_q[rs] = rstd_k[rs] = 1.f;
        }
    }
    __syncthreads();
    if (tid >= 128) {   // later row segments add the totals of the earlier ones
        const int d = tid & 127, part = tid >> 7;
        float t0 = 0.f;
        for (int q = 0; q < part; ++q) t0 += sHalf[q * DK + d];
#pragma unroll 8
        for (int r = 0; r < 64 / NPART; ++r) sG[(part * (64 / NPART) + r) * DK + d] += t0;
    }
    __syncthreads();
    if (tid < DK) reinterpret_cast<float*>(tile + TP_DECAY)[tid] = fast_exp2(sG[63 * DK + tid]);

    // ---- 3. operand generation + Gram MMAs, one 64-channel half at a time ----
    uint2 xpk[RS][4];
#pragma unroll 1
    for (int hf = 0; hf < 2; ++hf) {       // rolled: register arrays are picked with selects on static indices
        if (hf == 1) {   // operand buffers are reused: wait until the first half's MMAs have read them
            if (!mbar_wait(&bars[0], par)) atomicExch(p.status, STATUS_WAIT_TIMEOUT);
            umma::fence_after_sync();
        }
#pragma unroll
        for (int rs = 0; rs < RS; ++rs) {
            const int row = rq + RSTEP * rs, I = row >> 4, r7 = row & 7;
#pragma unroll
            for (int it = 0; it < 2; ++it) {
                const int grp = hf * 2 + it, d0 = 32 * grp + 4 * l8;
                const float4 Gi = *reinterpret_cast<const float4*>(sG + row * DK + d0);
                const float4 rI = *reinterpret_cast<const float4*>(sG + 16 * I * DK + d0);
                const float4 gL = *reinterpret_cast<const float4*>(sG + 63 * DK + d0);
                const float gi[4] = {Gi.x, Gi.y, Gi.z, Gi.w}, ri[4] = {rI.x, rI.y, rI.z, rI.w};
                const float gl[4] = {gL.x, gL.y, gL.z, gL.w};
                float qv[4], kv[4];
                {
                    const uint2 qsel = hf ? qraw[rs][2 + it] : qraw[rs][it];
                    const uint2 ksel = hf ? kraw[rs][2 + it] : kraw[rs][it];
                    float2 a = unpack_bf16(qsel.x), b = unpack_bf16(qsel.y);
                    qv[0] = a.x * rstd_q[rs]; qv[1] = a.y * rstd_q[rs]; qv[2] = b.x * rstd_q[rs]; qv[3] = b.y * rstd_q[rs];
                    a = unpack_bf16(ksel.x); b = unpack_bf16(ksel.y);
                    kv[0] = a.x * rstd_k[rs]; kv[1] = a.y * rstd_k[rs]; kv[2] = b.x * rstd_k[rs]; kv[3] = b.y * rstd_k[rs];
                }
                float qa[4], ka[4], kown[4], kg[4], qg[4], xx[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float eA = fast_exp2(gi[e] - ri[e]);      // <= 1
                    const float eB = fast_exp2(fminf(ri[e] - gi[e], 120.f));   // >= 1, <= 2^116 under the safe gate; the clamp
                                                                               // keeps an unbounded gate from making inf * 0
                    const float eG = fast_exp2(gi[e]);              // 2^(g_i)
                    qa[e] = qv[e] * eA;
                    ka[e] = kv[e] * eA;
                    kown[e] = kv[e] * eB;
                    kg[e] = kv[e] * fast_exp2(gl[e] - gi[e]);
                    qg[e] = p.scale * qv[e] * eG;
                    xx[e] = bet[rs] * kv[e] * eG;
                }
                const uint32_t sw = (uint32_t)((l8 ^ r7) << 4);
                unsigned char* opa = sm + SM_OPA + it * KATOM_A + sw;
                unsigned char* opb = sm + SM_OPB + it * KATOM_B + sw;
                *reinterpret_cast<float4*>(opa + row * 128) = tf32x4(qa[0], qa[1], qa[2], qa[3]);
                *reinterpret_cast<float4*>(opa + (row + 64) * 128) = tf32x4(ka[0], ka[1], ka[2], ka[3]);
                *reinterpret_cast<float4*>(opb + (8 * I * (I + 1) + row) * 128) = tf32x4(kown[0], kown[1], kown[2], kown[3]);
#pragma unroll
                for (int Ip = 1; Ip < 4; ++Ip) {
                    if (Ip > I) {     // copy anchored at the first row of the later block Ip: factor 2^(r_Ip - g_j) <= 1
                        const float4 rp = *reinterpret_cast<const float4*>(sG + 16 * Ip * DK + d0);
                        *reinterpret_cast<float4*>(opb + (8 * Ip * (Ip + 1) + row) * 128) =
                            tf32x4(kv[0] * fast_exp2(rp.x - gi[0]), kv[1] * fast_exp2(rp.y - gi[1]),
                                   kv[2] * fast_exp2(rp.z - gi[2]), kv[3] * fast_exp2(rp.w - gi[3]));
                    }
                }
                const int goff = swz256(row, d0);
                *reinterpret_cast<uint2*>(tile + TP_KG + goff) = make_uint2(pack_f16(kg[0], kg[1]), pack_f16(kg[2], kg[3]));
                *reinterpret_cast<uint2*>(tile + TP_QG + goff) = make_uint2(pack_f16(qg[0], qg[1]), pack_f16(qg[2], qg[3]));
                const uint2 xv = make_uint2(pack_f16(xx[0], xx[1]), pack_f16(xx[2], xx[3]));
                if (hf) xpk[rs][2 + it] = xv; else xpk[rs][it] = xv;
            }
        }
        fence_proxy_async();
        umma::fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            umma::fence_after_sync();
            const uint32_t idesc = umma::make_idesc(umma::FMT_TF32, 128, 160, false, false);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint64_t ad = sdesc_sw128(sm_u32 + SM_OPA + (ks >> 2) * KATOM_A + (ks & 3) * 32, 16, 1024);
                const uint64_t bd = sdesc_sw128(sm_u32 + SM_OPB + (ks >> 2) * KATOM_B + (ks & 3) * 32, 16, 1024);
                umma::mma_tf32(tmem, ad, bd, idesc, (hf | ks) != 0);
            }
            umma::commit(&bars[hf]);
        }
    }
    if (!mbar_wait(&bars[1], par)) atomicExch(p.status, STATUS_WAIT_TIMEOUT);
    umma::fence_after_sync();

    // ---- 4. X and Y = beta v into shared memory (all threads); Gram epilogue: warp w reads TMEM lane
    //         quadrant w&3 and handles the 16-row block (w&1)*2 + (w>>2) living in its lower/upper half ----
#pragma unroll
    for (int rs = 0; rs < RS; ++rs) {
        const int row = rq + RSTEP * rs;
#pragma unroll
        for (int grp = 0; grp < 4; ++grp) {
            const int chunk = 4 * (grp & 1) + (l8 >> 1);
            *reinterpret_cast<uint2*>(sm + SM_XS + (grp >> 1) * 8192 + row * 128 + ((chunk ^ (row & 7)) << 4) + (l8 & 1) * 8) =
                xpk[rs][grp];
        }
    }
    if (tile_id + (int)gridDim.x < p.num_tiles) fetch_rows(tile_id + gridDim.x);   // lands during the epilogues
    float* sL = reinterpret_cast<float*>(sm + SM_LF);
    float* sAi = reinterpret_cast<float*>(sm + SM_AINV);
    float* sT = reinterpret_cast<float*>(sm + SM_TM);
    {
        const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(p.v);
        uint4 raw[NIT];
#pragma unroll
        for (int n = 0; n < NIT; ++n) {
            const int idx = tid + INTRA_THREADS * n, j = idx >> 4, ch = idx & 15;
            raw[n] = make_uint4(0, 0, 0, 0);
            if (j < ci.valid) raw[n] = *reinterpret_cast<const uint4*>(vp + base + (size_t)j * tok_stride + 8 * ch);
        }
        {
            const int qd = warp & 3, bsel = (warp >> 2) & 1, gpar = warp >> 3;   // gpar splits the column groups (16 warps)
            const int blk = (qd & 1) * 2 + bsel;            // 16-row block handled by this warp
            const int row = (qd & 1) * 32 + lane;           // row of this lane inside the 64-row matrix
            const bool mine = (row >> 4) == blk;
            const bool is_q = qd < 2;                       // lanes 0..63 hold q rows (-> Aqk), 64..127 k rows (-> L)
            const float bi = sBeta[row];
            const uint32_t taddr = tmem + ((uint32_t)(qd * 32) << 16) + 8 * blk * (blk + 1);
#pragma unroll 1
            for (int gcol = gpar; gcol < 4; gcol += NWARPS / 8) {
                if (gcol > blk) {                            // warp-uniform: nothing but zeros right of the block
                    if (mine && is_q) {
                        *reinterpret_cast<uint4*>(tile + TP_AQK + swz128(row, 16 * gcol)) = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(tile + TP_AQK + swz128(row, 16 * gcol + 8)) = make_uint4(0, 0, 0, 0);
                    }
                    continue;
                }
                uint32_t r[16];
                umma::ld_32x32b_x16(taddr + 16 * gcol, r);
                umma::wait_ld();
                if (mine) {
                    float vals[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const int j = 16 * gcol + e;
                        const float x = __uint_as_float(r[e]);
                        vals[e] = is_q ? ((j <= row) ? p.scale * x : 0.f) : ((j < row) ? bi * x : 0.f);
                    }
                    if (is_q) {
#pragma unroll
                        for (int hc = 0; hc < 2; ++hc)
                            *reinterpret_cast<uint4*>(tile + TP_AQK + swz128(row, 16 * gcol + 8 * hc)) =
                                make_uint4(pack_f16(vals[8 * hc], vals[8 * hc + 1]), pack_f16(vals[8 * hc + 2], vals[8 * hc + 3]),
                                           pack_f16(vals[8 * hc + 4], vals[8 * hc + 5]), pack_f16(vals[8 * hc + 6], vals[8 * hc + 7]));
                    } else {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4)
                            *reinterpret_cast<float4*>(sL + row * LROW + 16 * gcol + 4 * q4) =
                                make_float4(vals[4 * q4], vals[4 * q4 + 1], vals[4 * q4 + 2], vals[4 * q4 + 3]);
                        if (p.mkk_out) {     // the same Gram entries without beta, for the backward pass
                            float* mo = p.mkk_out + ((size_t)c * p.H + h) * BT * BT + row * BT + 16 * gcol;
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) {
                                float mv[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const int j = 16 * gcol + 4 * q4 + e;
                                    mv[e] = (j < row) ? __uint_as_float(r[4 * q4 + e]) : 0.f;
                                }
                                *reinterpret_cast<float4*>(mo + 4 * q4) = make_float4(mv[0], mv[1], mv[2], mv[3]);
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int n = 0; n < NIT; ++n) {
            const int idx = tid + INTRA_THREADS * n, j = idx >> 4, ch = idx & 15;
            const float b = sBeta[j];
            const uint32_t w4[4] = {raw[n].x, raw[n].y, raw[n].z, raw[n].w};
            uint32_t o4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float2 f = unpack_bf16(w4[e]);
                o4[e] = pack_f16(b * f.x, b * f.y);
            }
            *reinterpret_cast<uint4*>(sm + SM_YS + (ch >> 3) * 8192 + j * 128 + (((ch & 7) ^ (j & 7)) << 4)) =
                make_uint4(o4[0], o4[1], o4[2], o4[3]);
        }
    }
    umma::fence_before_sync();
    __syncthreads();

    // ---- 5. Akk = (I + L)^-1: 16x16 diagonal blocks by substitution (64 threads; the others clear the
    //         blocks above the diagonal), then 16->32->64 block merges X = -D2inv (C D1inv) as split-TF32
    //         mma.sync products (three MMAs per step recover fp32-level accuracy) ----
    if (tid < 64) {
        const int b = tid >> 4, cc = tid & 15;
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float acc = (i == cc) ? 1.f : 0.f;
#pragma unroll
            for (int j = 0; j < i; ++j) acc = fmaf(-sL[(16 * b + i) * LROW + 16 * b + j], x[j], acc);
            x[i] = acc;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) sAi[(16 * b + i) * LROW + 16 * b + cc] = x[i];
    } else if (tid < 192) {   // zero blocks (0,1) and (2,3): they are read as part of the 32x32 factors
        const int t = tid - 64, pr = t >> 6, i = (t >> 2) & 15, j4 = (t & 3) * 4;
        *reinterpret_cast<float4*>(sAi + (32 * pr + i) * LROW + 32 * pr + 16 + j4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncthreads();
    {
        const int g8 = lane >> 2, t4 = lane & 3;
        // level 1: pairs pr = 0,1 -> block (2pr+1, 2pr). T = C * D1inv, one 16x8 tile per warp 0..3
        if (warp < 4) {
            const int pr = warp >> 1, nt = warp & 1, r0 = 32 * pr + 16, c0 = 32 * pr;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            mma_tile_3xtf32<2>(sL + r0 * LROW + c0, LROW, sAi + c0 * LROW + c0 + 8 * nt, LROW, acc, g8, t4);
            float* td = sT + (16 * pr) * TROW + 8 * nt;
            td[g8 * TROW + 2 * t4] = acc[0]; td[g8 * TROW + 2 * t4 + 1] = acc[1];
            td[(g8 + 8) * TROW + 2 * t4] = acc[2]; td[(g8 + 8) * TROW + 2 * t4 + 1] = acc[3];
        }
        __syncthreads();
        if (warp < 4) {
            const int pr = warp >> 1, nt = warp & 1, r0 = 32 * pr + 16, c0 = 32 * pr;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            mma_tile_3xtf32<2>(sAi + r0 * LROW + r0, LROW, sT + (16 * pr) * TROW + 8 * nt, TROW, acc, g8, t4);
            float* xd = sAi + r0 * LROW + c0 + 8 * nt;
            xd[g8 * LROW + 2 * t4] = -acc[0]; xd[g8 * LROW + 2 * t4 + 1] = -acc[1];
            xd[(g8 + 8) * LROW + 2 * t4] = -acc[2]; xd[(g8 + 8) * LROW + 2 * t4 + 1] = -acc[3];
        }
        __syncthreads();
        // level 2: block rows 32..63 x cols 0..31. One 16x8 tile per warp (2 m-tiles x 4 n-tiles)
        const int mt = (warp >> 2) & 1, nt = warp & 3;
        if (warp < 8) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            mma_tile_3xtf32<4>(sL + (32 + 16 * mt) * LROW, LROW, sAi + 8 * nt, LROW, acc, g8, t4);
            float* td = sT + (16 * mt) * TROW + 8 * nt;
            td[g8 * TROW + 2 * t4] = acc[0]; td[g8 * TROW + 2 * t4 + 1] = acc[1];
            td[(g8 + 8) * TROW + 2 * t4] = acc[2]; td[(g8 + 8) * TROW + 2 * t4 + 1] = acc[3];
        }
        __syncthreads();
        if (warp < 8) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            mma_tile_3xtf32<4>(sAi + (32 + 16 * mt) * LROW + 32, LROW, sT + 8 * nt, TROW, acc, g8, t4);
            float* xd = sAi + (32 + 16 * mt) * LROW + 8 * nt;
            xd[g8 * LROW + 2 * t4] = -acc[0]; xd[g8 * LROW + 2 * t4 + 1] = -acc[1];
            xd[(g8 + 8) * LROW + 2 * t4] = -acc[2]; xd[(g8 + 8) * LROW + 2 * t4 + 1] = -acc[3];
        }
    }
    __syncthreads();
    {   // Akk -> fp16 K-major operand (and fp32 to HBM when the backward pass wants it)
        constexpr int CPT = 4096 / INTRA_THREADS;              // columns per thread: 16 or 8
        const int row = tid / (64 / CPT), c0 = (tid % (64 / CPT)) * CPT;
        float v[CPT];
#pragma unroll
        for (int e = 0; e < CPT; ++e) {
            const int j = c0 + e;
            v[e] = (j <= row) ? sAi[row * LROW + j] : 0.f;
        }
#pragma unroll
        for (int hc = 0; hc < CPT / 8; ++hc) {
            const int ch = (c0 >> 3) + hc;
            const uint4 pk = make_uint4(pack_f16(v[8 * hc], v[8 * hc + 1]), pack_f16(v[8 * hc + 2], v[8 * hc + 3]),
                                        pack_f16(v[8 * hc + 4], v[8 * hc + 5]), pack_f16(v[8 * hc + 6], v[8 * hc + 7]));
            unsigned char* dstk = sm + SM_AKK16 + row * 128 + ((ch ^ (row & 7)) << 4);
            *reinterpret_cast<uint4*>(dstk) = pk;
            *reinterpret_cast<uint4*>(dstk + 8192) = pk;        // rows 64..127 of the A operand repeat Akk
        }
        if (p.akk_out) {
            float* ao = p.akk_out + ((size_t)c * p.H + h) * BT * BT + row * BT + c0;
#pragma unroll
            for (int q4 = 0; q4 < CPT / 4; ++q4)
                *reinterpret_cast<float4*>(ao + 4 * q4) = make_float4(v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]);
        }
    }
    fence_proxy_async();
    umma::fence_before_sync();
    __syncthreads();

    // ---- 6. [w | u] = Akk [X | Y]: one M=128 x N=256 x K=64 product. A = Akk stacked twice (K-major), so TMEM
    //         lanes 0..63 and 64..127 both hold the 64 token rows; B = [X | Y] as four MN-major 64-channel atoms ----
    if (tid == 0) {
        umma::fence_after_sync();
        const uint32_t idesc = umma::make_idesc(umma::FMT_F16, 128, 256, false, true);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint64_t ad = sdesc_sw128(sm_u32 + SM_AKK16 + ks * 32, 16, 1024);
            const uint64_t bd = sdesc_sw128(sm_u32 + SM_XS + ks * 2048, 8192, 1024);
            umma::mma_f16(tmem, ad, bd, idesc, ks != 0);
        }
        umma::commit(&bars[2]);
    }
    if (!mbar_wait(&bars[2], par)) atomicExch(p.status, STATUS_WAIT_TIMEOUT);
    umma::fence_after_sync();

    // ---- 7. epilogue: lane = token, columns = channels; lanes 0..63 write w, the duplicate lanes 64..127 write u;
    //         each thread converts 64/(NWARPS/8) channels to fp16 and stores 16 bytes at a time ----
    {
        const int qd = warp & 3, is_u = qd >> 1, tok = 32 * (qd & 1) + lane;
        constexpr int CPW = 512 / NWARPS;                      // channels per warp: 64 (8 warps) or 32 (16 warps)
        const int ch0 = (warp >> 2) * CPW;                     // first channel (0..127) of this warp
        const uint32_t taddr = tmem + ((uint32_t)(32 * qd) << 16) + 128 * is_u + ch0;
        bool out_of_range = false;
#pragma unroll 1
        for (int cg = 0; cg < CPW / 16; ++cg) {
            uint32_t r[16];
            umma::ld_32x32b_x16(taddr + 16 * cg, r);
            umma::wait_ld();
            const int chn = ch0 + 16 * cg;
#pragma unroll
            for (int hc = 0; hc < 2; ++hc) {
                const uint4 pk = make_uint4(pack_f16(__uint_as_float(r[8 * hc]), __uint_as_float(r[8 * hc + 1])),
                                            pack_f16(__uint_as_float(r[8 * hc + 2]), __uint_as_float(r[8 * hc + 3])),
                                            pack_f16(__uint_as_float(r[8 * hc + 4]), __uint_as_float(r[8 * hc + 5])),
                                            pack_f16(__uint_as_float(r[8 * hc + 6]), __uint_as_float(r[8 * hc + 7])));
                out_of_range |= f16x2_not_finite(pk.x) | f16x2_not_finite(pk.y) | f16x2_not_finite(pk.z) | f16x2_not_finite(pk.w);
                const int cc = chn + 8 * hc;
                if (is_u) *reinterpret_cast<uint4*>(tile + (cc < 64 ? TP_U0 : TP_U1) + swz128(tok, cc & 63)) = pk;
                else *reinterpret_cast<uint4*>(tile + TP_W + swz256(tok, cc)) = pk;
            }
        }
        // w and u inherit the range of v and of (I + L)^-1: fp16 has no room beyond 65504, so say so instead of
        // handing inf to the scan
        if (__any_sync(0xffffffffu, out_of_range) && lane == 0) atomicMax(p.status, STATUS_RANGE);
    }
    umma::fence_before_sync();
    __syncthreads();      // TMEM columns and shared memory are free for the next tile
    umma::fence_after_sync();
    }  // tile loop
    if (warp == 0) umma::tmem_dealloc(tmem, 256);
}

}  // namespace kda

extern "C" int kda_fwd_intra_smem_bytes() { return kda::SM_TOTAL + 1024; }

extern "C" int kda_launch_fwd_intra(const kda::IntraParams* p, int num_chunks, cudaStream_t stream) {
    using namespace kda;
    if (num_chunks <= 0) return 0;
    const int smem = SM_TOTAL + 1024;
    cudaError_t e = cudaFuncSetAttribute(kda_fwd_intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    IntraParams q = *p;
    q.num_tiles = num_chunks * p->H;
    const int grid = q.num_tiles < 2 * sms ? q.num_tiles : 2 * sms;     // two resident CTAs per SM
    kda_fwd_intra_kernel<<<grid, INTRA_THREADS, smem, stream>>>(q);
    return (int)cudaGetLastError();
}
