// Chunk-parallel forward stage on tcgen05 tensor cores: one CTA per (chunk, head) fuses
//   gate activation + per-chunk cumulative sum (log2 domain), q/k L2 normalisation,
//   the gated 64x64 Gram matrices Aqk / L (one M=128 x N=160 TF32 UMMA chain, accumulators in TMEM),
//   Akk = (I + L)^-1 (blocked 16 -> 32 -> 64 inverse in fp32),
//   [w | u] = Akk [beta k 2^g | beta v] (two M=128 x N=128 FP16 UMMA chains),
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
// 2^(r_I - g_j), which is <= 1 for earlier blocks and at most 2^(16*5*log2 e) ~ 2^116 inside block I.
// So the B operand holds one copy of k-hat per anchor: 16 + 32 + 48 + 64 = 160 rows; the A operand
// is [q-hat ; k-hat] scaled by their own block anchors (128 rows). Column block I of the 128 x 160
// product is valid on the rows of block I only; the epilogue reads exactly those.
// Every factor is built from TWO exponentials per element, 2^(g_i - r_I) and 2^(r_{I+1} - g_i), times constants that
// depend on (block, channel) only and are tabulated once per tile (phase 3 below).
//
// Two CTAs are resident per SM (110 KB shared memory, 256 TMEM columns each), so one CTA's CUDA-core
// operand generation overlaps the other's MMA, inverse and epilogues.
#include "kda_common.cuh"
#include "kda_params.h"
#include "umma.cuh"

// Optional per-phase cycle counters (compile with -DKDA_PHASE_TIMERS): thread 0 of every CTA adds the clock64() spent
// between consecutive marks to a device array that kda_fwd_intra_read_timers() copies out (profiling builds only).
#ifdef KDA_PHASE_TIMERS
__device__ unsigned long long kda_fwd_intra_timers[16];
#define PHASE_MARK(i)                                                                     \
    do {                                                                                  \
        if (tid == 0) {                                                                   \
            const long long now_ = clock64();                                             \
            atomicAdd(&kda_fwd_intra_timers[i], (unsigned long long)(now_ - phase_t0_));  \
            phase_t0_ = now_;                                                             \
        }                                                                                 \
    } while (0)
#else
#define PHASE_MARK(i) do {} while (0)
#endif

namespace kda {

constexpr int INTRA_THREADS = 256;              // 8 warps; warp w owns token rows 8w .. 8w+7 in the first phases
constexpr int NWARPS = INTRA_THREADS / 32;
constexpr int NIT = 1024 / INTRA_THREADS;        // (row, 16-lane) items per thread when v is staged
constexpr int INFO_THREAD = 224;                 // the thread that works out the next tile's geometry

// shared-memory map (bytes from a 1024-aligned base)
constexpr int SM_OPA = 0;                 // A operand of one 64-channel half: [2 k-atoms][128 rows][128 B], SW128
constexpr int SM_OPB = 32768;             // B operand: [2 k-atoms][160 rows][128 B], SW128
constexpr int SM_XS = 73728;              // X = beta k 2^g, fp16 [2 mn-atoms][64 tokens][128 B], SW128 (MN-major B operand)
constexpr int SM_MISC = 90112;            // per-tile scalars (beta[2][64], alpha[2], dt_bias[2][128]: this tile's and the
                                          // next tile's), barriers, tmem base, abort flag
constexpr int SM_BIAS = SM_MISC + 1024;   // [2][128] fp32
constexpr int SM_TOT = SM_MISC + 2048;    // [8][128] fp32: sum of the log2 decays of each 8-row group
constexpr int SM_A16 = SM_TOT + 4096;     // [4][128] fp32: log2 decay of the first row of each 16-row block
// per-channel tables built once per tile from the two arrays above (by 128 threads, one channel each)
constexpr int SM_PRE = SM_A16 + 2048;     // [8][128] sum of the groups before group w
constexpr int SM_R = SM_PRE + 4096;       // [5][128] r_0..r_3: cumulative log2 decay at the first row of each block; r_4 = g_last
constexpr int SM_CG = SM_R + 2560;        // [4][128] 2^(r_I)
constexpr int SM_CB = SM_CG + 2048;       // [4][128] 2^(r_I - r_{I+1})
constexpr int SM_CK = SM_CB + 2048;       // [4][128] 2^(g_last - r_{I+1})
constexpr int SM_C2 = SM_CK + 2048;       // [128]    2^(r_2 - r_1)
constexpr int SM_C3 = SM_C2 + 512;        // [2][128] 2^(r_3 - r_{I+1}), I = 0, 1
constexpr int SM_TOTAL = SM_C3 + 1024;
constexpr int KATOM_A = 16384, KATOM_B = 20480;
// regions reused once the Gram MMAs have completed
constexpr int SM_YS = SM_OPA;             // Y = beta v, same layout as X
constexpr int LROW = 68;                  // padded fp32 row of the 64x64 matrices
constexpr int SM_LF = SM_OPB;             // L fp32 [64][68]
constexpr int SM_AINV = SM_OPB + 17408;   // (I+L)^-1 fp32 [64][68]
constexpr int SM_TM = SM_OPB + 34816;     // scratch for the block products [32][36]
constexpr int TROW = 36;
// staging of the lane-per-token outputs: written in the exact tile-pack image, then sent to HBM by bulk copies (one
// thread, asynchronous) instead of 16-byte stores that hit a different 128-byte line in every lane
constexpr int SM_STG_AQK = SM_OPA + 16384;   // [64][128 B]: free from the Gram epilogue on (Y only takes the first 16 KB)
constexpr int SM_STG_U = SM_OPA;             // U0 | U1, [2][64][128 B]: Y is dead once the W/U MMAs have completed
constexpr int SM_STG_W = SM_XS;              // [64][256 B]: so is X
constexpr int SM_AKK16 = SM_LF;           // Akk fp16, stacked twice: [128][128 B], SW128 (K-major A operand); L is dead by then
static_assert(SM_TM + 32 * TROW * 4 <= SM_XS, "inverse scratch must fit the B operand region");


__device__ __forceinline__ uint64_t sdesc_sw128(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return umma::make_sdesc(addr, lbo, sbo) | (2ull << 61);
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
    hi = (__float_as_uint(x) + 0x1000u) & 0xffffe000u;                 // nearest, ties away (what cvt.rna.tf32 gives)
    lo = __float_as_uint(x - __uint_as_float(hi)) & 0xffffe000u;       // the residual: truncation is enough
}
__device__ __forceinline__ void mma_tf32_16x8x8(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
template <int KT>
__device__ __forceinline__ void mma_tile_3xtf32(const float* A, int lda, const float* B, int ldb, float (&acc)[4], int g, int t) {
#pragma unroll
    for (int ks = 0; ks < KT; ++ks) {      // unrolled: the loads of all k-steps are in flight together (a latency chain otherwise)
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

// ---- packed fp32 pairs (one instruction per two lanes of arithmetic on sm_100) ----
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 r;
    asm("{.reg .b64 ra, rb, rc; mov.b64 ra, {%2, %3}; mov.b64 rb, {%4, %5}; mul.rn.f32x2 rc, ra, rb; mov.b64 {%0, %1}, rc;}"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 r;
    asm("{.reg .b64 ra, rb, rc; mov.b64 ra, {%2, %3}; mov.b64 rb, {%4, %5}; add.rn.f32x2 rc, ra, rb; mov.b64 {%0, %1}, rc;}"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 r;
    asm("{.reg .b64 ra, rb, rc, rd; mov.b64 ra, {%2, %3}; mov.b64 rb, {%4, %5}; mov.b64 rc, {%6, %7}; "
        "fma.rn.f32x2 rd, ra, rb, rc; mov.b64 {%0, %1}, rd;}"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return r;
}
__device__ __forceinline__ float2 sub2(float2 a, float2 b) { return add2(a, make_float2(-b.x, -b.y)); }
__device__ __forceinline__ float2 ex2_2(float2 a) { return make_float2(fast_exp2(a.x), fast_exp2(a.y)); }
__device__ __forceinline__ float2 splat2(float a) { return make_float2(a, a); }
// The tensor core reads only the upper 19 bits of a tf32 operand, i.e. it truncates. Instead of rounding every
// operand (one more instruction per element), the mean relative error of truncation, -0.5 ulp * E[1/mantissa] =
// -2^-11 / ln 2 = -3.52e-4 for log-uniform mantissas, is compensated once per operand SIDE by scaling both gate factors
// by (1 + 3.52e-4): the shift TF32_DEBIAS_LOG2 is folded into the exponents of eA and f below, and its inverse into
// the table constants of the fp16 outputs (kg, qg, x), which must not carry it. Measured on N(0,1) and U(0,1) rows,
// weak and strong gates: (I + L)^-1 and Aqk are as accurate as with round-to-nearest operands (7e-5 / 3e-4 relative),
// three to six times better than plain truncation.
constexpr float TF32_DEBIAS_LOG2 = 5.0775e-4f;          // log2(1 + 3.52e-4)
constexpr float TF32_DEBIAS_INV = 0.99964812f;          // 1 / (1 + 3.52e-4)
__device__ __forceinline__ float4 tf32x4(float2 a, float2 b) { return make_float4(a.x, a.y, b.x, b.y); }
__device__ __forceinline__ uint2 f16x4(float2 a, float2 b) { return make_uint2(pack_f16(a.x, a.y), pack_f16(b.x, b.y)); }

__global__ void __launch_bounds__(INTRA_THREADS, 2) kda_fwd_intra_kernel(const IntraParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sm_u32 = smem_u32(sm);
    float* sBetaBuf = reinterpret_cast<float*>(sm + SM_MISC);            // [2][64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + SM_MISC + 512);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + SM_MISC + 544);
    volatile int* sAbort = reinterpret_cast<volatile int*>(sm + SM_MISC + 552);
    float* sAlpha = reinterpret_cast<float*>(sm + SM_MISC + 560);        // [2] exp(A_log[h])
    int4* sInfo = reinterpret_cast<int4*>(sm + SM_MISC + 576);           // [2] {first token row, valid rows, head, tile slot}
    float* sBiasBuf = reinterpret_cast<float*>(sm + SM_BIAS);            // [2][128]
    float* sTot = reinterpret_cast<float*>(sm + SM_TOT);
    float* sA16 = reinterpret_cast<float*>(sm + SM_A16);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t tok_stride = (size_t)p.H * DK;
    // first phases: warp w owns rows 8w..8w+7 (all of them in 16-row block I = w / 2); lane (r2, cq) owns rows
    // 8w + 4 r2 + j, j = 0..3, and channels 64 hf + 4 cq + e, e = 0..3, of both 64-channel halves hf
    const int r2 = lane >> 4, cq = lane & 15, I = warp >> 1, row0 = 8 * warp + 4 * r2;

    if (tid == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_init(&bars[2], 1);
        *sAbort = 0;
        fence_mbar_init();
    }
    if (warp == 0) umma::tmem_alloc(tmem_slot, 256);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    // the state scan that follows in the stream may be scheduled as soon as SMs free up, so that its launch and set-up
    // run under the tail of this kernel; it waits for this whole grid before it reads anything
    pdl_launch_dependents();
#ifdef KDA_PHASE_TIMERS
    long long phase_t0_ = clock64();
#endif

    // One thread waits (bounded) for the tensor-core completion barrier; everybody else parks on the CTA barrier.
    // On a time-out the status word is set and the whole CTA leaves the tile loop together (TMEM is freed below).
    auto wait_mma = [&](int which, uint32_t parity) -> bool {
        if (tid == 0) {
            if (!mbar_wait(&bars[which], parity)) {
                atomicExch(p.status, STATUS_WAIT_TIMEOUT);
                *sAbort = 1;
            }
            umma::fence_before_sync();
        }
        __syncthreads();
        umma::fence_after_sync();
        return *sAbort == 0;
    };

    // The geometry of a tile (integer divisions, table look-ups for a packed batch) is worked out by ONE thread, one
    // tile ahead, and handed to the others through shared memory.
    auto publish_info = [&](int t_id, int buf) {
        if (tid == INFO_THREAD) {
            int4 v = make_int4(0, 0, 0, 0);
            if (t_id < p.num_tiles) {
                const int c2 = t_id / p.H;
                const ChunkInfo ci2 = chunk_info(c2, p.cu_seqlens, p.chunk_indices, p.T);
                v = make_int4(ci2.row0, ci2.valid, t_id - c2 * p.H, t_id);
            }
            sInfo[buf] = v;
        }
    };
    // Register prefetch: the raw gate rows are fetched one tile ahead (they are the first thing a tile needs); q and k
    // rows are fetched at the top of their own tile and first used after the gate phase, from L2 (see l2_hints).
    // Loads are unconditional (nothing may depend on a loaded value before it is used): a padding row reads the last
    // real row of the chunk instead, and is zeroed where it is used (through its gate, norm and beta factors).
    uint2 qraw[4][2], kraw[4][2], graw[4][2];     // [row j][half]: 4 bf16 each; fp32 gates are loaded in place instead
    auto fetch_g = [&](const int4 nf) {
        if (p.g_fp32 || p.g_per_head) return;
        const __nv_bfloat16* gp = reinterpret_cast<const __nv_bfloat16*>(p.g) + (size_t)nf.x * tok_stride + (size_t)nf.z * DK + 4 * cq;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const size_t roff = (size_t)min(row0 + j, nf.y - 1) * tok_stride;
            graw[j][0] = *reinterpret_cast<const uint2*>(gp + roff);
            graw[j][1] = *reinterpret_cast<const uint2*>(gp + roff + 64);
        }
    };
    auto fetch_qk = [&](const int4 nf) {
        const size_t base2 = (size_t)nf.x * tok_stride + (size_t)nf.z * DK + 4 * cq;
        const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(p.q) + base2;
        const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(p.k) + base2;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const size_t roff = (size_t)min(row0 + j, nf.y - 1) * tok_stride;
            qraw[j][0] = *reinterpret_cast<const uint2*>(qp + roff);
            qraw[j][1] = *reinterpret_cast<const uint2*>(qp + roff + 64);
            kraw[j][0] = *reinterpret_cast<const uint2*>(kp + roff);
            kraw[j][1] = *reinterpret_cast<const uint2*>(kp + roff + 64);
        }
    };
    // Per-tile scalars (beta of the 64 rows, dt_bias and exp(A_log) of the head) are fetched one tile ahead by the
    // first 129 threads into a register each and parked in shared memory before the tile ends, so that no phase of
    // the next tile starts with a dependent global load.
    uint32_t sc_next = 0;        // raw bits: nothing may depend on the load before it is parked
    auto load_scalars = [&](const int4 nf) {
        const int h2 = nf.z;
        sc_next = 0;
        if (tid < BT) {
            if (tid < nf.y) {
                const size_t bi = (size_t)(nf.x + tid) * p.H + h2;
                sc_next = p.beta_fp32 ? reinterpret_cast<const uint32_t*>(p.beta)[bi]
                                      : (uint32_t)reinterpret_cast<const uint16_t*>(p.beta)[bi];
            }
        } else if (tid < BT + DK) {
            if (p.gate_mode != GATE_NONE && p.dt_bias) sc_next = __float_as_uint(p.dt_bias[h2 * DK + tid - BT]);
        } else if (tid == BT + DK) {
            if (p.gate_mode != GATE_NONE) sc_next = __float_as_uint(p.A_log[h2]);
        }
    };
    auto park_scalars = [&](int buf, int valid_rows) {
        if (tid < BT) {
            float b = p.beta_fp32 ? __uint_as_float(sc_next) : __uint_as_float(sc_next << 16);
            if (p.beta_logit) b = (tid < valid_rows) ? __fdividef(1.f, 1.f + __expf(-b)) : 0.f;    // padding rows stay 0
            sBetaBuf[buf * BT + tid] = b;
        }
        else if (tid < BT + DK) sBiasBuf[buf * DK + tid - BT] = __uint_as_float(sc_next);
        else if (tid == BT + DK) sAlpha[buf] = p.gate_mode != GATE_NONE ? __expf(__uint_as_float(sc_next)) : 0.f;
    };
    publish_info(blockIdx.x, 0);
    __syncthreads();
    if ((int)blockIdx.x < p.num_tiles) {
        fetch_g(sInfo[0]);
        load_scalars(sInfo[0]);
        park_scalars(0, sInfo[0].y);
    }
    __syncthreads();

    // persistent over (chunk, head) tiles; the completion barriers flip phase once per tile
    for (int tile_id = blockIdx.x, iter = 0; tile_id < p.num_tiles; tile_id += gridDim.x, ++iter) {
    const uint32_t par = iter & 1;
    const float* sBeta = sBetaBuf + par * BT;
    const int4 info = sInfo[par];
    struct { int row0, valid; } ci = {info.x, info.y};
    const int h = info.z;
    const size_t base = (size_t)ci.row0 * tok_stride + (size_t)h * DK;
    unsigned char* tile = p.tiles + (size_t)tile_id * TP_BYTES;       // tile slot = chunk * H + head = tile_id
    publish_info(tile_id + gridDim.x, par ^ 1);      // visible to everybody after the next barrier
    fetch_qk(info);

    // the gate rows of this tile are already in registers: they were fetched while the previous tile was in its
    // epilogues (first tile: before the loop).
    auto l2_hints = [&]() {   // pull this tile's v rows and the next tile's inputs towards L2 (two 128-byte lines per row)
        const int row = tid >> 2, part = tid & 3;
        if (part < 2 && row < ci.valid)
            prefetch_l2(reinterpret_cast<const __nv_bfloat16*>(p.v) + base + (size_t)row * tok_stride + 64 * part);
        const int4 nf = sInfo[par ^ 1];
        if (nf.y > 0) {
            struct { int row0, valid; } ni = {nf.x, nf.y};
            const int nh = nf.z;
            if (row < ni.valid) {
                const size_t nb = (size_t)(ni.row0 + row) * tok_stride + (size_t)nh * DK + 64 * (part & 1);
                if (part < 2) {
                    prefetch_l2(reinterpret_cast<const __nv_bfloat16*>(p.q) + nb);
                    prefetch_l2(reinterpret_cast<const __nv_bfloat16*>(p.k) + nb);
                } else if (p.g_per_head) {
                    // a few bytes per row: not worth a hint
                } else if (p.g_fp32) {
                    prefetch_l2(reinterpret_cast<const float*>(p.g) + nb);
                    prefetch_l2(reinterpret_cast<const float*>(p.g) + nb + 32);
                } else {
                    prefetch_l2(reinterpret_cast<const __nv_bfloat16*>(p.g) + nb);
                }
            }
        }
    };
    // ---- 1. gate activation (log2 domain) and the cumulative sum over the thread's four rows, then over the
    //         warp's eight rows with one exchange between the two lane halves; padding rows contribute 0 ----
    float2 G[4][4];            // [row j][pair]: pairs 0,1 = channels 4cq..4cq+3, pairs 2,3 = 64+4cq..64+4cq+3
    {
        PHASE_MARK(15);                 // what the compiler placed at the top of a tile (index and address arithmetic)
        const float alpha = sAlpha[par];
        float2 bias[4];
        {
            const float4 b0 = *reinterpret_cast<const float4*>(sBiasBuf + par * DK + 4 * cq);
            const float4 b1 = *reinterpret_cast<const float4*>(sBiasBuf + par * DK + 64 + 4 * cq);
            bias[0] = make_float2(b0.x, b0.y); bias[1] = make_float2(b0.z, b0.w);
            bias[2] = make_float2(b1.x, b1.y); bias[3] = make_float2(b1.z, b1.w);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const bool live = row0 + j < ci.valid;
            float2 gv[4];
            if (p.g_per_head) {        // one gate per (token, head): every channel gets the same value
                float gs = 0.f;
                if (live) {
                    const size_t gi = (size_t)(ci.row0 + row0 + j) * p.H + h;
                    gs = p.g_fp32 ? reinterpret_cast<const float*>(p.g)[gi]
                                  : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.g)[gi]);
                }
                gv[0] = gv[1] = gv[2] = gv[3] = make_float2(gs, gs);
            } else if (p.g_fp32) {
                float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
                if (live) {
                    const float* gp = reinterpret_cast<const float*>(p.g) + base + (size_t)(row0 + j) * tok_stride + 4 * cq;
                    lo = *reinterpret_cast<const float4*>(gp);
                    hi = *reinterpret_cast<const float4*>(gp + 64);
                }
                gv[0] = make_float2(lo.x, lo.y); gv[1] = make_float2(lo.z, lo.w);
                gv[2] = make_float2(hi.x, hi.y); gv[3] = make_float2(hi.z, hi.w);
            } else {
                gv[0] = unpack_bf16(graw[j][0].x); gv[1] = unpack_bf16(graw[j][0].y);
                gv[2] = unpack_bf16(graw[j][1].x); gv[3] = unpack_bf16(graw[j][1].y);
            }
            if (p.gate_mode == GATE_LOWER_BOUND) {
                // lower_bound * sigmoid(alpha x) / ln2 with one ex2 and one rcp per element (flush-to-zero approximations)
                const float2 c0 = splat2(-alpha * RCP_LN2), c1 = splat2(live ? p.lower_bound * RCP_LN2 : 0.f);
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float2 e = add2(ex2_2(mul2(c0, add2(gv[x], bias[x]))), splat2(1.f));
                    G[j][x] = mul2(c1, make_float2(fast_rcp(e.x), fast_rcp(e.y)));
                }
            } else {
                const float keep = live ? RCP_LN2 : 0.f;
#pragma unroll
                for (int x = 0; x < 4; ++x)
                    G[j][x] = make_float2(keep * gate_activation(gv[x].x, alpha, bias[x].x, p.gate_mode, p.lower_bound),
                                          keep * gate_activation(gv[x].y, alpha, bias[x].y, p.gate_mode, p.lower_bound));
            }
        }
        PHASE_MARK(0); // gate activation
#pragma unroll
        for (int j = 1; j < 4; ++j)
#pragma unroll
            for (int x = 0; x < 4; ++x) G[j][x] = add2(G[j][x], G[j - 1][x]);
        float2 oth[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            oth[x].x = __shfl_xor_sync(0xffffffffu, G[3][x].x, 16);
            oth[x].y = __shfl_xor_sync(0xffffffffu, G[3][x].y, 16);
        }
        if (r2 == 0) {       // group total and, for the first warp of a 16-row block, the value at the block's first row
            float* td = sTot + warp * DK + 4 * cq;
            *reinterpret_cast<float4*>(td) = make_float4(G[3][0].x + oth[0].x, G[3][0].y + oth[0].y, G[3][1].x + oth[1].x, G[3][1].y + oth[1].y);
            *reinterpret_cast<float4*>(td + 64) = make_float4(G[3][2].x + oth[2].x, G[3][2].y + oth[2].y, G[3][3].x + oth[3].x, G[3][3].y + oth[3].y);
            if ((warp & 1) == 0) {
                float* ad = sA16 + I * DK + 4 * cq;
                *reinterpret_cast<float4*>(ad) = make_float4(G[0][0].x, G[0][0].y, G[0][1].x, G[0][1].y);
                *reinterpret_cast<float4*>(ad + 64) = make_float4(G[0][2].x, G[0][2].y, G[0][3].x, G[0][3].y);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int x = 0; x < 4; ++x) G[j][x] = add2(G[j][x], oth[x]);
        }
    }
    PHASE_MARK(2);      // in-warp cumulative sum, totals
    // ---- 2. L2 norms of the thread's four q and k rows (sum over the 16 lanes that share the rows), beta ----
    float rstd_q[4], rstd_k[4], bet[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float2 sq = make_float2(0.f, 0.f), sk = sq;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            float2 a = unpack_bf16(qraw[j][hf].x), b = unpack_bf16(qraw[j][hf].y);
            sq = fma2(a, a, sq); sq = fma2(b, b, sq);
            a = unpack_bf16(kraw[j][hf].x); b = unpack_bf16(kraw[j][hf].y);
            sk = fma2(a, a, sk); sk = fma2(b, b, sk);
        }
        bet[j] = sBeta[row0 + j];
        if (p.use_l2norm) {
            float s1 = sq.x + sq.y, s2 = sk.x + sk.y;
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) {
                s1 += __shfl_xor_sync(0xffffffffu, s1, o);
                s2 += __shfl_xor_sync(0xffffffffu, s2, o);
            }
            rstd_q[j] = rsqrtf(s1 + 1e-6f);
            rstd_k[j] = rsqrtf(s2 + 1e-6f);
        } else {
            rstd_q[j] = rstd_k[j] = 1.f;
        }
        if (row0 + j >= ci.valid) rstd_q[j] = rstd_k[j] = 0.f;      // padding rows: q = k = 0
    }
    PHASE_MARK(14);     // norms, beta
    __syncthreads();          // group totals and block-start values are visible
    PHASE_MARK(1);      // barrier
    if (tid < DK) {
        // one channel per thread: prefix sums of the group totals, the block anchors, and every per-(block, channel)
        // constant of the operand generation below (15 exponentials per channel instead of several per element)
        float run = 0.f, P[NWARPS];
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            P[w] = run;
            reinterpret_cast<float*>(sm + SM_PRE)[w * DK + tid] = run;
            run += sTot[w * DK + tid];
        }
        const float r[5] = {sA16[tid], P[2] + sA16[DK + tid], P[4] + sA16[2 * DK + tid], P[6] + sA16[3 * DK + tid], run};
        reinterpret_cast<float*>(tile + TP_DECAY)[tid] = fast_exp2(run);      // 2^(g_last): the decay of the whole chunk
#pragma unroll
        for (int b = 0; b < 5; ++b) reinterpret_cast<float*>(sm + SM_R)[b * DK + tid] = r[b];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            reinterpret_cast<float*>(sm + SM_CG)[b * DK + tid] = TF32_DEBIAS_INV * fast_exp2(r[b]);
            // >= 1, <= 2^116 under the safe gate; the clamp keeps an unbounded gate from making inf * 0
            reinterpret_cast<float*>(sm + SM_CB)[b * DK + tid] = fast_exp2(fminf(r[b] - r[b + 1], 126.f));
            reinterpret_cast<float*>(sm + SM_CK)[b * DK + tid] = TF32_DEBIAS_INV * fast_exp2(run - r[b + 1]);
        }
        reinterpret_cast<float*>(sm + SM_C2)[tid] = fast_exp2(r[2] - r[1]);
        reinterpret_cast<float*>(sm + SM_C3)[tid] = fast_exp2(r[3] - r[1]);
        reinterpret_cast<float*>(sm + SM_C3)[DK + tid] = fast_exp2(r[3] - r[2]);
    }
    if (tid == 0) bulk_wait_read_all();   // the previous tile's staged outputs have left the operand buffers
    __syncthreads();          // tables are visible
    PHASE_MARK(2);      // tables (same slot as the in-warp scan)

    // ---- 3. operand generation + Gram MMAs, one 64-channel half at a time. Per element only two exponentials:
    //         eA = 2^(g_i - r_I) and f = 2^(r_N - g_i) (r_I: log2 decay at the first row of the element's 16-row
    //         block, r_N: at the first row of the next block, or g_last for the last block; both factors <= 1).
    //         Every other factor is one of them times a per-(block, channel) constant from the tables:
    //           2^(g_i)        = eA 2^(r_I)               -> qg, x
    //           2^(r_I - g_i)  = f 2^(r_I - r_N)          -> own-block copy of the B operand
    //           2^(g_last-g_i) = f 2^(g_last - r_N)       -> kg
    //           2^(r_J - g_i)  = f 2^(r_J - r_N), J > I+1 -> copies anchored at later blocks ----
#pragma unroll 1
    for (int hf = 0; hf < 2; ++hf) {       // rolled: register arrays are picked with selects on static indices
        if (hf == 1 && !wait_mma(0, par)) break;   // operand buffers are reused: the first half's MMAs must have read them
        if (hf == 1) PHASE_MARK(4);                // MMA issue + wait for the first half
        // rI, rN: the two anchors minus the sum of the groups before this warp's rows, so that they can be compared
        // with the thread's group-local cumulative sums directly
        float2 rI[2], rN[2], cG[2], cB[2], cK[2], c2[2], c3[2];
        {
            const int co = 64 * hf + 4 * cq;
            auto ld = [&](int off, float2 (&dst)[2]) {
                const float4 t = *reinterpret_cast<const float4*>(sm + off + 4 * co);
                dst[0] = make_float2(t.x, t.y); dst[1] = make_float2(t.z, t.w);
            };
            float2 pre[2];
            ld(SM_PRE + warp * DK * 4, pre);
            ld(SM_R + I * DK * 4, rI);
            ld(SM_R + (I + 1) * DK * 4, rN);
            ld(SM_CG + I * DK * 4, cG);
            ld(SM_CB + I * DK * 4, cB);
            ld(SM_CK + I * DK * 4, cK);
            ld(SM_C2, c2);                            // used by block 0 only
            ld(SM_C3 + (I & 1) * DK * 4, c3);         // used by blocks 0 and 1
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                rI[x] = sub2(rI[x], add2(pre[x], splat2(TF32_DEBIAS_LOG2)));       // eA = 2^(g - rI) carries (1 + 3.52e-4)
                rN[x] = sub2(rN[x], add2(pre[x], splat2(-TF32_DEBIAS_LOG2)));      // and so does f = 2^(rN - g)
            }
        }
        const int atom = cq >> 3;
        unsigned char* opa = sm + SM_OPA + atom * KATOM_A;
        unsigned char* opb = sm + SM_OPB + atom * KATOM_B;
        unsigned char* xs = sm + SM_XS + hf * 8192;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int row = row0 + j;
            const uint32_t sw = (uint32_t)(((cq & 7) ^ (row & 7)) << 4);
            const uint2 qsel = hf ? qraw[j][1] : qraw[j][0];
            const uint2 ksel = hf ? kraw[j][1] : kraw[j][0];
            const float2 gi[2] = {hf ? G[j][2] : G[j][0], hf ? G[j][3] : G[j][1]};     // group-local cumulative sums
            const float2 rq2 = splat2(rstd_q[j]), rk2 = splat2(rstd_k[j]);
            const float2 qh[2] = {mul2(unpack_bf16(qsel.x), rq2), mul2(unpack_bf16(qsel.y), rq2)};
            const float2 kh[2] = {mul2(unpack_bf16(ksel.x), rk2), mul2(unpack_bf16(ksel.y), rk2)};
            float2 qa[2], ka[2], ko[2], kg[2], qg[2], xx[2], kf[2], k2[2], k3[2];
            const float2 sc2 = splat2(p.scale), be2 = splat2(bet[j]);
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const float2 eA = ex2_2(sub2(gi[x], rI[x]));      // <= 1
                const float2 f = ex2_2(sub2(rN[x], gi[x]));       // <= 1
                qa[x] = mul2(qh[x], eA);
                ka[x] = mul2(kh[x], eA);
                kf[x] = mul2(kh[x], f);                           // k 2^(r_N - g_i): the copy anchored at the next block
                ko[x] = mul2(kf[x], cB[x]);
                kg[x] = mul2(kf[x], cK[x]);
                k2[x] = mul2(kf[x], c2[x]);
                k3[x] = mul2(kf[x], c3[x]);
                const float2 qG = mul2(qa[x], cG[x]);             // q 2^(g_i)
                qg[x] = mul2(qG, sc2);
                xx[x] = mul2(mul2(ka[x], cG[x]), be2);
            }
            *reinterpret_cast<float4*>(opa + row * 128 + sw) = tf32x4(qa[0], qa[1]);
            *reinterpret_cast<float4*>(opa + (row + 64) * 128 + sw) = tf32x4(ka[0], ka[1]);
            *reinterpret_cast<float4*>(opb + (8 * I * (I + 1) + row) * 128 + sw) = tf32x4(ko[0], ko[1]);
            // copies anchored at the first row of the later blocks: factor 2^(r_J - g_i) <= 1
            if (I < 3) *reinterpret_cast<float4*>(opb + (8 * (I + 1) * (I + 2) + row) * 128 + sw) = tf32x4(kf[0], kf[1]);
            if (I == 0) *reinterpret_cast<float4*>(opb + (8 * 2 * 3 + row) * 128 + sw) = tf32x4(k2[0], k2[1]);
            if (I < 2) *reinterpret_cast<float4*>(opb + (8 * 3 * 4 + row) * 128 + sw) = tf32x4(k3[0], k3[1]);
            const int goff = swz256(row, 64 * hf + 4 * cq);
            *reinterpret_cast<uint2*>(tile + TP_KG + goff) = f16x4(kg[0], kg[1]);
            *reinterpret_cast<uint2*>(tile + TP_QG + goff) = f16x4(qg[0], qg[1]);
            // X = beta k 2^g as the MN-major B operand of the W/U product: [token][64 channels of this half], SW128
            *reinterpret_cast<uint2*>(xs + row * 128 + ((((cq >> 1) ^ (row & 7))) << 4) + (cq & 1) * 8) = f16x4(xx[0], xx[1]);
        }
        fence_proxy_async();
        umma::fence_before_sync();
        __syncthreads();
        PHASE_MARK(3 + 2 * hf);      // operand generation of this half (3, 5)
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
        if (hf == 0) l2_hints();          // while the first half's MMAs run
    }
    // ---- 4. Y = beta v into shared memory (all threads); Gram epilogue: warp w reads TMEM lane
    //         quadrant w&3 and handles the 16-row block (w&1)*2 + (w>>2) living in its lower/upper half ----
    // While the second half's MMAs run: issue the loads whose results are needed later -- the next tile's gate rows
    // and scalars (they land during the epilogues) and this tile's v rows.
    if (!*sAbort && tile_id + (int)gridDim.x < p.num_tiles) {
        fetch_g(sInfo[par ^ 1]);
        load_scalars(sInfo[par ^ 1]);
    }
    float* sL = reinterpret_cast<float*>(sm + SM_LF);
    float* sAi = reinterpret_cast<float*>(sm + SM_AINV);
    float* sT = reinterpret_cast<float*>(sm + SM_TM);
    uint4 raw[NIT];
    {
        const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(p.v);
#pragma unroll
        for (int n = 0; n < NIT; ++n) {
            const int idx = tid + INTRA_THREADS * n, j = idx >> 4, ch = idx & 15;
            // a padding row reads the last real row; its beta is 0, so Y = beta v is 0 there
            raw[n] = *reinterpret_cast<const uint4*>(vp + base + (size_t)min(j, ci.valid - 1) * tok_stride + 8 * ch);
        }
    }
    PHASE_MARK(12);     // next tile's loads and this tile's v loads issued
    if (*sAbort || !wait_mma(1, par)) break;
    PHASE_MARK(6);      // wait for the second half's MMAs
    {
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
                        *reinterpret_cast<uint4*>(sm + SM_STG_AQK + swz128(row, 16 * gcol)) = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(sm + SM_STG_AQK + swz128(row, 16 * gcol + 8)) = make_uint4(0, 0, 0, 0);
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
                            *reinterpret_cast<uint4*>(sm + SM_STG_AQK + swz128(row, 16 * gcol + 8 * hc)) =
                                make_uint4(pack_f16(vals[8 * hc], vals[8 * hc + 1]), pack_f16(vals[8 * hc + 2], vals[8 * hc + 3]),
                                           pack_f16(vals[8 * hc + 4], vals[8 * hc + 5]), pack_f16(vals[8 * hc + 6], vals[8 * hc + 7]));
                    } else {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4)
                            *reinterpret_cast<float4*>(sL + row * LROW + 16 * gcol + 4 * q4) =
                                make_float4(vals[4 * q4], vals[4 * q4 + 1], vals[4 * q4 + 2], vals[4 * q4 + 3]);
                        if (p.mkk_out) {     // the same Gram entries without beta, for the backward pass
                            float* mo = p.mkk_out + (size_t)tile_id * BT * BT + row * BT + 16 * gcol;
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
        PHASE_MARK(13);     // Gram epilogue
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
    park_scalars(par ^ 1, sInfo[par ^ 1].y);
    umma::fence_before_sync();
    __syncthreads();
    PHASE_MARK(7);      // v loads, Gram epilogue, Y staging

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
    PHASE_MARK(8);      // triangular inverse
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
            float* ao = p.akk_out + (size_t)tile_id * BT * BT + row * BT + c0;
#pragma unroll
            for (int q4 = 0; q4 < CPT / 4; ++q4)
                *reinterpret_cast<float4*>(ao + 4 * q4) = make_float4(v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]);
        }
    }
    fence_proxy_async();
    umma::fence_before_sync();
    __syncthreads();

    // ---- 6. [w | u] = Akk [X | Y]: two M=128 x N=128 x K=64 products into TMEM columns 0..127 (w) and 128..255 (u).
    //         A = Akk stacked twice (K-major), so TMEM lanes 0..63 and 64..127 both hold the 64 token rows;
    //         B = X, then Y, each as two MN-major 64-channel atoms ----
    if (tid == 0) {
        umma::fence_after_sync();
        const uint32_t idesc = umma::make_idesc(umma::FMT_F16, 128, 128, false, true);
#pragma unroll
        for (int part = 0; part < 2; ++part) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ad = sdesc_sw128(sm_u32 + SM_AKK16 + ks * 32, 16, 1024);
                const uint64_t bd = sdesc_sw128(sm_u32 + (part ? SM_YS : SM_XS) + ks * 2048, 8192, 1024);
                umma::mma_f16(tmem + 128 * part, ad, bd, idesc, ks != 0);
            }
        }
        umma::commit(&bars[2]);
    }
    PHASE_MARK(9);      // Akk pack + W/U MMA issue
    if (!wait_mma(2, par)) break;
    PHASE_MARK(10);     // W/U MMA wait

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
                if (is_u) *reinterpret_cast<uint4*>(sm + SM_STG_U + (cc < 64 ? 0 : 8192) + swz128(tok, cc & 63)) = pk;
                else *reinterpret_cast<uint4*>(sm + SM_STG_W + swz256(tok, cc)) = pk;
            }
        }
        // w and u inherit the range of v and of (I + L)^-1: fp16 has no room beyond 65504, so say so instead of
        // handing inf to the scan
        if (__any_sync(0xffffffffu, out_of_range) && lane == 0) atomicMax(p.status, STATUS_RANGE);
    }
    fence_proxy_async();
    umma::fence_before_sync();
    __syncthreads();      // TMEM columns are free for the next tile; the staged outputs are complete
    umma::fence_after_sync();
    if (tid == 0) {       // w, u and Aqk leave as three bulk copies; their buffers are next written by the operand generation
        bulk_s2g(tile + TP_W, sm + SM_STG_W, 16384);
        bulk_s2g(tile + TP_U0, sm + SM_STG_U, 16384);
        bulk_s2g(tile + TP_AQK, sm + SM_STG_AQK, 8192);
        bulk_commit();
    }
    PHASE_MARK(11);     // W/U epilogue
    }  // tile loop
    if (tid == 0) bulk_wait_all();        // staged outputs must be on their way before the shared memory goes away
    if (warp == 0) umma::tmem_dealloc(tmem, 256);
}

}  // namespace kda

extern "C" int kda_fwd_intra_smem_bytes() { return kda::SM_TOTAL + 1024; }

#ifdef KDA_PHASE_TIMERS
extern "C" int kda_fwd_intra_read_timers(unsigned long long* out, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out, kda_fwd_intra_timers, sizeof(kda_fwd_intra_timers));
    if (e == cudaSuccess && reset) {
        unsigned long long z[16] = {};
        e = cudaMemcpyToSymbol(kda_fwd_intra_timers, z, sizeof(z));
    }
    return (int)e;
}
#endif

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
