// Sequential state scan fused with the output stage.
//
// One CTA per (sequence, head, half of the value columns). Four consumer warps each own 16 value
// columns of the fp32 state, held TRANSPOSED in mma.sync accumulator registers (S^T: 16 x 128 per
// warp) for the whole sequence: because the accumulator fragment of one m16n8k16 MMA is exactly the
// A fragment of the next, the chain
//     v_new^T = u^T - S^T w^T ;  o^T = S^T qg^T + v_new^T Aqk^T ;  S^T <- S^T diag(decay) + v_new^T kg
// runs without the state ever leaving registers and without any cross-warp synchronisation. A fifth
// warp is the producer: it streams the per-chunk tile packs through a 3-stage shared-memory ring
// with bulk (TMA-engine) copies signalled on mbarriers.
//
// Replaces chunk_gated_delta_rule_fwd_h (cula/ops/chunk_delta_h.py:1991-2168) and chunk_gla_fwd_o
// (cula/ops/fwd_o.py:1755-1852); the per-chunk states h and v_new only go to HBM when the caller
// asks for them (backward recomputation, return_intermediate_states).
#include "kda_common.cuh"
#include "kda_params.h"

namespace kda {

constexpr int SCAN_STAGES = 3;
constexpr int SCAN_STAGE_BYTES = TP_HEAD_BYTES + 8192;   // W,QG,KG,AQK,DECAY + one U half = 66048
constexpr int SCAN_STG_BYTES = 4096;                     // per-warp staging for coalesced stores
constexpr int SCAN_CONSUMERS = 4;
constexpr int SCAN_THREADS = (SCAN_CONSUMERS + 1) * 32;
constexpr int SCAN_SMEM = SCAN_STAGES * SCAN_STAGE_BYTES + SCAN_CONSUMERS * SCAN_STG_BYTES + 64;
constexpr int ST_U = TP_HEAD_BYTES;                      // offset of the U half inside a stage

// Shared-memory layout of a pipeline stage. The full scan stages the whole head of a tile pack plus one U half and
// runs one CTA per SM; the transition scan needs only W, KG, DECAY and the U half, packs them tightly, keeps two
// stages (the producer warp pulls the chunks after those into L2) and so fits two CTAs per SM.
// NVH = value halves per CTA. 1: a CTA carries 64 value columns on 4 consumer warps (grid.x = 2), three stages.
// 2: both halves on 8 consumer warps (two per scheduler, so one warp's dependent chain fills the other's bubbles in
// the tensor pipe), the whole tile pack per stage, two stages; used when there are more scan CTAs than SMs.
template <bool TRANSITION, int NVH>
struct ScanLayout {
    static constexpr int CONSUMERS = SCAN_CONSUMERS * NVH;
    static constexpr int STAGES = NVH == 2 ? 2 : SCAN_STAGES, STAGE_BYTES = TP_HEAD_BYTES + 8192 * NVH;
    static constexpr int W = TP_W, KG = TP_KG, DECAY = TP_DECAY, U = ST_U;
    static constexpr int STG = CONSUMERS * SCAN_STG_BYTES;
    static constexpr int SMEM = STAGES * STAGE_BYTES + STG + 64;
    static constexpr int CTAS_PER_SM = 1;
};
template <>
struct ScanLayout<true, 1> {
    static constexpr int CONSUMERS = SCAN_CONSUMERS;
    static constexpr int STAGES = 2;
    static constexpr int W = 0, KG = 16384, DECAY = 32768, U = 33280, STAGE_BYTES = 41472;
    static constexpr int STG = 0;
    static constexpr int SMEM = STAGES * STAGE_BYTES + STG + 64;
    static constexpr int CTAS_PER_SM = 2;
};

// Bounded wait that also ends when *votes reaches `quorum` (the CTA has nothing left to compute).
// Returns 0 = barrier phase completed, 1 = gave up (time-out), 2 = quorum reached.
__device__ __forceinline__ int mbar_wait_or_quorum(uint64_t* bar, uint32_t parity, volatile int* votes, int quorum) {
    for (int i = 0; i < (1 << 22); ++i) {
        if (mbar_test(bar, parity)) return 0;
        if (*votes >= quorum) return 2;
        if (i > 64) __nanosleep(64);
    }
    return 1;
}

// TRANSITION: the affine action of a whole shard on the state, S_out = M S_in + C, from the same recurrence with
// four column groups per (sequence, head): groups 0,1 carry C (zero start, normal u; written to p.ht) and groups
// 2,3 carry the K x K matrix M = prod_c (D_c - kg_c^T w_c) (identity start, u = 0; written to p.m_out). No output
// rows are produced. Used by context parallelism.
template <bool STORE_HV, bool TRANSITION, int NVH = 1>
__global__ void __launch_bounds__((SCAN_CONSUMERS * NVH + 1) * 32, ScanLayout<TRANSITION, NVH>::CTAS_PER_SM)
kda_fwd_scan_kernel(const ScanParams p) {
    static_assert(NVH == 1 || !TRANSITION, "both value halves per CTA: not for the transition scan");
    using L = ScanLayout<TRANSITION, NVH>;
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::STAGES * L::STAGE_BYTES + L::STG);
    uint64_t* empty = full + L::STAGES;
    // Columns of the transition matrix M that have become exactly zero stay zero (their recurrence is linear and has
    // no source term), so a warp whose 16 columns are all zero votes once and stops computing; when all consumer warps
    // of an M-carrying CTA have voted, the CTA is finished -- bit-identical results, and with strong gates (the decay
    // of one chunk underflows fp32) these CTAs free their SMs for the C-carrying ones after a chunk or two.
    volatile int* zero_votes = reinterpret_cast<volatile int*>(empty + L::STAGES);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // Grid: (column group, head, sequence). When the transition scan has more CTAs than SMs it is launched as
    // (head, sequence, column group) instead: block indices are handed to the SMs in linear order, so all C-carrying
    // CTAs (groups 0, 1) come first, one per SM, and the M-carrying ones (groups 2, 3) become their co-residents; when
    // the M CTAs finish early (see zero_votes) every C CTA is left with an SM of its own. (With fewer CTAs than SMs the
    // original order keeps the four CTAs of a head on neighbouring SMs, which read the same tile packs.)
    const bool gm = TRANSITION && p.group_major;
    const int cgrp = gm ? blockIdx.z : blockIdx.x, seq_slot = gm ? blockIdx.y : blockIdx.z;
    const bool is_m = TRANSITION && cgrp >= 2;           // this CTA carries columns of M
    const int vh = NVH == 2 ? ((warp >> 2) & 1) : (cgrp & 1), h = gm ? blockIdx.x : blockIdx.y;
    const int pw = warp & 3;                             // 16-column slice of the value half
    const int n = p.seq_order ? p.seq_order[seq_slot] : seq_slot;
    int bos, len, chunk0;
    if (p.cu_seqlens) {
        bos = p.cu_seqlens[n];
        len = p.cu_seqlens[n + 1] - bos;
        chunk0 = p.chunk_offsets[n];
    } else {
        bos = n * p.T;
        len = p.T;
        chunk0 = n * ((p.T + BT - 1) / BT);
    }
    const int nchunks = (len + BT - 1) / BT;

    if (tid == 0) {
        for (int s = 0; s < L::STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], L::CONSUMERS);
        }
        *zero_votes = 0;
        fence_mbar_init();
    }
    __syncthreads();
    // Everything this kernel reads (tile packs, initial states) may come from the kernels before it in the stream; with
    // programmatic stream serialization the CTA can be resident before they have finished, so wait here (a no-op when
    // the launch does not carry the attribute). Only scheduling, the index arithmetic and the barrier set-up above overlap.
    pdl_wait();

    if (warp == L::CONSUMERS) {
        // ------------------------------- producer warp -------------------------------
        if (TRANSITION) {
            const int u_off = vh ? TP_U1 : TP_U0;
            int issued = 0;                       // chunks whose copies have been issued
            for (int c = 0; c < nchunks; ++c) {
                const int s = c % L::STAGES, use = c / L::STAGES;
                bool ok = true;
                int quorum = 0;
                if (lane == 0) {
                    if (is_m && *zero_votes >= L::CONSUMERS) quorum = 1;
                    if (!quorum && use > 0) {
                        const int r = mbar_wait_or_quorum(&empty[s], (use - 1) & 1, zero_votes, is_m ? L::CONSUMERS : (1 << 30));
                        ok = r != 1;
                        quorum = r == 2;
                    }
                }
                quorum = __shfl_sync(0xffffffffu, quorum, 0);
                if (quorum) break;
                if (lane == 0) {
                    if (ok) {
                        const unsigned char* tile = p.tiles + ((size_t)(chunk0 + c) * p.H + h) * TP_BYTES;
                        unsigned char* dst = smem + s * L::STAGE_BYTES;
                        mbar_arrive_expect_tx(&full[s], is_m ? L::U : L::STAGE_BYTES);
                        bulk_g2s(dst + L::W, tile + TP_W, 16384, &full[s]);
                        bulk_g2s(dst + L::KG, tile + TP_KG, 16384, &full[s]);
                        bulk_g2s(dst + L::DECAY, tile + TP_DECAY, 512, &full[s]);
                        if (!is_m) bulk_g2s(dst + L::U, tile + u_off, 8192, &full[s]);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    if (lane == 0) atomicExch(p.status, STATUS_WAIT_TIMEOUT);
                    break;
                }
                issued = c + 1;
                const int cn = c + L::STAGES;                 // not yet being copied: pull it into L2
                if (cn < nchunks) {
                    const unsigned char* tile = p.tiles + ((size_t)(chunk0 + cn) * p.H + h) * TP_BYTES;
                    for (int i = lane; i < (is_m ? 260 : 324); i += 32) {
                        const int off = i < 128 ? TP_W + i * 128 : i < 256 ? TP_KG + (i - 128) * 128
                                      : i < 260 ? TP_DECAY + (i - 256) * 128 : u_off + (i - 260) * 128;
                        prefetch_l2(tile + off);
                    }
                }
            }
            // the consumers may have left early: do not exit with bulk copies to this CTA's shared memory in flight
            if (is_m && lane == 0) {
                for (int cc = max(0, issued - L::STAGES); cc < issued; ++cc)
                    if (!mbar_wait(&full[cc % L::STAGES], (cc / L::STAGES) & 1)) atomicExch(p.status, STATUS_WAIT_TIMEOUT);
            }
            return;
        }
        if (lane == 0) {
            for (int c = 0; c < nchunks; ++c) {
                const int s = c % L::STAGES, use = c / L::STAGES;
                if (use > 0 && !mbar_wait(&empty[s], (use - 1) & 1)) {
                    atomicExch(p.status, STATUS_WAIT_TIMEOUT);
                    break;
                }
                const unsigned char* tile = p.tiles + ((size_t)(chunk0 + c) * p.H + h) * TP_BYTES;
                unsigned char* dst = smem + s * L::STAGE_BYTES;
                mbar_arrive_expect_tx(&full[s], L::STAGE_BYTES);
                if (NVH == 2) {
                    bulk_g2s(dst, tile, TP_BYTES, &full[s]);          // head + both U halves are contiguous
                } else {
                    bulk_g2s(dst, tile, TP_HEAD_BYTES, &full[s]);
                    bulk_g2s(dst + ST_U, tile + ((cgrp & 1) ? TP_U1 : TP_U0), 8192, &full[s]);
                }
            }
        }
        return;
    }

    // ---------------------------------- consumer warps ----------------------------------
    const int g = lane >> 2, t = lane & 3;
    const int m = lane >> 3, r = lane & 7;          // ldmatrix/stmatrix: matrix index, row inside it
    const int vb = vh * 64 + pw * 16;               // first value column of this warp
    unsigned char* stg = smem + L::STAGES * L::STAGE_BYTES + warp * SCAN_STG_BYTES;   // unused by the transition scan
    const uint32_t stg_u32 = smem_u32(stg);

    float S[16][4];
    if (is_m) {
#pragma unroll
        for (int jt = 0; jt < 16; ++jt) {
            const int k0 = 8 * jt + 2 * t;
            S[jt][0] = (k0 == vb + g) ? 1.f : 0.f;
            S[jt][1] = (k0 + 1 == vb + g) ? 1.f : 0.f;
            S[jt][2] = (k0 == vb + g + 8) ? 1.f : 0.f;
            S[jt][3] = (k0 + 1 == vb + g + 8) ? 1.f : 0.f;
        }
    } else if (!TRANSITION && p.h0) {
        const float* h0 = p.h0 + ((size_t)n * p.H + h) * DK * DV;
#pragma unroll
        for (int jt = 0; jt < 16; ++jt) {
            int k0 = 8 * jt + 2 * t;
            S[jt][0] = h0[(size_t)k0 * DV + vb + g];
            S[jt][1] = h0[(size_t)(k0 + 1) * DV + vb + g];
            S[jt][2] = h0[(size_t)k0 * DV + vb + g + 8];
            S[jt][3] = h0[(size_t)(k0 + 1) * DV + vb + g + 8];
        }
    } else {
#pragma unroll
        for (int jt = 0; jt < 16; ++jt) S[jt][0] = S[jt][1] = S[jt][2] = S[jt][3] = 0.f;
    }

    // per-lane swizzled column-group offsets for the four k-step pairs of a 256-byte-row operand
    uint32_t x256[4];
#pragma unroll
    for (int kp = 0; kp < 4; ++kp) x256[kp] = (uint32_t)(((4 * kp + m) ^ r) << 4);

    bool voted = false;          // this warp's columns of M are exactly zero (transition scan only)
    for (int c = 0; c < nchunks; ++c) {
        const int s = c % L::STAGES;
        if (is_m) {
            if (*zero_votes >= L::CONSUMERS) break;
            const int r = mbar_wait_or_quorum(&full[s], (c / L::STAGES) & 1, zero_votes, L::CONSUMERS);
            if (r == 2) break;
            if (r == 1) {
                atomicExch(p.status, STATUS_WAIT_TIMEOUT);
                return;
            }
            if (voted) {         // nothing to compute: keep the pipeline protocol going for the warps that still work
                if (lane == 0) mbar_arrive(&empty[s]);
                continue;
            }
        } else if (!mbar_wait(&full[s], (c / L::STAGES) & 1)) {
            atomicExch(p.status, STATUS_WAIT_TIMEOUT);
            return;
        }
        const uint32_t st = smem_u32(smem + s * L::STAGE_BYTES);
        const int valid = min(BT, len - c * BT);
        const size_t tile_idx = (size_t)(chunk0 + c) * p.H + h;

        // ---- S as fp16 A fragments (8 k-steps over the 128 key channels), scaled by a per-warp power
        //      of two so that the largest entry sits near 2^13: fp16 then carries 11 significant bits
        //      whatever the magnitude of the state, and cannot overflow ----
        float smax = 0.f;
#pragma unroll
        for (int jt = 0; jt < 16; ++jt)
            smax = fmaxf(smax, fmaxf(fmaxf(fabsf(S[jt][0]), fabsf(S[jt][1])), fmaxf(fabsf(S[jt][2]), fabsf(S[jt][3]))));
#pragma unroll
        for (int o = 16; o; o >>= 1) smax = fmaxf(smax, __shfl_xor_sync(0xffffffffu, smax, o));
        if (is_m && smax == 0.f) {      // all 16 columns of this warp are exactly zero, and will stay zero
            voted = true;
            if (lane == 0) {
                atomicAdd(const_cast<int*>(zero_votes), 1);
                mbar_arrive(&empty[s]);
            }
            continue;
        }
        int shift = 13 - (((__float_as_int(smax) >> 23) & 0xff) - 127);
        shift = max(-100, min(100, shift));
        const float s_up = __int_as_float((shift + 127) << 23), s_down = __int_as_float((127 - shift) << 23);
        uint32_t sa[8][4];
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            sa[ks][0] = pack_f16(S[2 * ks][0] * s_up, S[2 * ks][1] * s_up);
            sa[ks][1] = pack_f16(S[2 * ks][2] * s_up, S[2 * ks][3] * s_up);
            sa[ks][2] = pack_f16(S[2 * ks + 1][0] * s_up, S[2 * ks + 1][1] * s_up);
            sa[ks][3] = pack_f16(S[2 * ks + 1][2] * s_up, S[2 * ks + 1][3] * s_up);
        }
        if (STORE_HV) {
            if (p.h_out) {
                // incoming state of this chunk, bf16 [128 k][128 v]; this warp owns a 32-byte column slice
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    int krow = 8 * (2 * ks + (m >> 1)) + r;
                    stsm_x4_t(stg_u32 + krow * 32 + (m & 1) * 16,
                              pack_bf16(S[2 * ks][0], S[2 * ks][1]), pack_bf16(S[2 * ks][2], S[2 * ks][3]),
                              pack_bf16(S[2 * ks + 1][0], S[2 * ks + 1][1]), pack_bf16(S[2 * ks + 1][2], S[2 * ks + 1][3]));
                }
                __syncwarp();
                unsigned char* hg = reinterpret_cast<unsigned char*>(p.h_out) + tile_idx * (size_t)(DK * DV * 2);
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    int row = it * 16 + (lane >> 1), hf = lane & 1;
                    uint4 val = *reinterpret_cast<const uint4*>(stg + row * 32 + hf * 16);
                    *reinterpret_cast<uint4*>(hg + (size_t)row * 256 + vb * 2 + hf * 16) = val;
                }
                __syncwarp();
            }
            if (p.h32_out) {
                // the same state in fp32 [128 k][128 v] for the backward pass
                float* hg = p.h32_out + tile_idx * (size_t)(DK * DV);
#pragma unroll
                for (int jt = 0; jt < 16; ++jt) {
                    int k0 = 8 * jt + 2 * t;
                    hg[(size_t)k0 * DV + vb + g] = S[jt][0];
                    hg[(size_t)(k0 + 1) * DV + vb + g] = S[jt][1];
                    hg[(size_t)k0 * DV + vb + g + 8] = S[jt][2];
                    hg[(size_t)(k0 + 1) * DV + vb + g + 8] = S[jt][3];
                }
            }
        }

        // ---- acc = S^T w^T : [16 v] x [64 tokens], contraction over 128 key channels ----
        float acc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
        for (int kp = 0; kp < 4; ++kp) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(st + L::W + (8 * nt + r) * 256 + x256[kp], b0, b1, b2, b3);
                mma_f16(acc[nt], sa[2 * kp], b0, b1);
                mma_f16(acc[nt], sa[2 * kp + 1], b2, b3);
            }
        }
        // ---- v_new^T = u^T - acc  (u = 0 for the transition matrix) ----
        if (is_m) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                acc[nt][0] *= -s_down; acc[nt][1] *= -s_down; acc[nt][2] *= -s_down; acc[nt][3] *= -s_down;
            }
        } else {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            uint32_t r0, r1, r2, r3;
            int row = 8 * (2 * np + (m >> 1)) + r, ch = 2 * pw + (m & 1);
            ldsm_x4_t(st + L::U + (NVH == 2 ? vh * 8192 : 0) + row * 128 + ((ch ^ r) << 4), r0, r1, r2, r3);
            float2 f;
            f = unpack_f16(r0); acc[2 * np][0] = fmaf(-s_down, acc[2 * np][0], f.x); acc[2 * np][1] = fmaf(-s_down, acc[2 * np][1], f.y);
            f = unpack_f16(r1); acc[2 * np][2] = fmaf(-s_down, acc[2 * np][2], f.x); acc[2 * np][3] = fmaf(-s_down, acc[2 * np][3], f.y);
            f = unpack_f16(r2); acc[2 * np + 1][0] = fmaf(-s_down, acc[2 * np + 1][0], f.x); acc[2 * np + 1][1] = fmaf(-s_down, acc[2 * np + 1][1], f.y);
            f = unpack_f16(r3); acc[2 * np + 1][2] = fmaf(-s_down, acc[2 * np + 1][2], f.x); acc[2 * np + 1][3] = fmaf(-s_down, acc[2 * np + 1][3], f.y);
        }
        }
        uint32_t va[4][4];   // v_new^T as fp16 A fragments (4 k-steps over the 64 tokens)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            va[ks][0] = pack_f16(acc[2 * ks][0], acc[2 * ks][1]);
            va[ks][1] = pack_f16(acc[2 * ks][2], acc[2 * ks][3]);
            va[ks][2] = pack_f16(acc[2 * ks + 1][0], acc[2 * ks + 1][1]);
            va[ks][3] = pack_f16(acc[2 * ks + 1][2], acc[2 * ks + 1][3]);
        }
        if (STORE_HV) {
            // v_new, fp16 [64 tokens][128 v]
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                int trow = 8 * (2 * ks + (m >> 1)) + r;
                stsm_x4_t(stg_u32 + trow * 32 + (m & 1) * 16, va[ks][0], va[ks][1], va[ks][2], va[ks][3]);
            }
            __syncwarp();
            unsigned char* vg = reinterpret_cast<unsigned char*>(p.vnew_out) + tile_idx * (size_t)(BT * DV * 2);
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                int row = it * 16 + (lane >> 1), hf = lane & 1;
                uint4 val = *reinterpret_cast<const uint4*>(stg + row * 32 + hf * 16);
                *reinterpret_cast<uint4*>(vg + (size_t)row * 256 + vb * 2 + hf * 16) = val;
            }
            __syncwarp();
        }

        // ---- o^T = S^T qg^T + v_new^T Aqk^T (skipped when no output is wanted: backward recomputation) ----
        if (!TRANSITION && (!STORE_HV || p.o != nullptr)) {
            float oacc[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) oacc[nt][0] = oacc[nt][1] = oacc[nt][2] = oacc[nt][3] = 0.f;
#pragma unroll
            for (int kp = 0; kp < 4; ++kp) {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(st + TP_QG + (8 * nt + r) * 256 + x256[kp], b0, b1, b2, b3);
                    mma_f16(oacc[nt], sa[2 * kp], b0, b1);
                    mma_f16(oacc[nt], sa[2 * kp + 1], b2, b3);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                oacc[nt][0] *= s_down; oacc[nt][1] *= s_down; oacc[nt][2] *= s_down; oacc[nt][3] *= s_down;
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int ksp = 0; ksp < 2; ++ksp) {
                    if (32 * ksp <= 8 * nt + 7) {      // causal: skip column blocks right of the diagonal
                        uint32_t b0, b1, b2, b3;
                        ldsm_x4(st + TP_AQK + (8 * nt + r) * 128 + (((4 * ksp + m) ^ r) << 4), b0, b1, b2, b3);
                        mma_f16(oacc[nt], va[2 * ksp], b0, b1);
                        if (32 * ksp + 16 <= 8 * nt + 7) mma_f16(oacc[nt], va[2 * ksp + 1], b2, b3);
                    }
                }
            }
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                int trow = 8 * (2 * np + (m >> 1)) + r;
                stsm_x4_t(stg_u32 + trow * 32 + (m & 1) * 16,
                          pack_bf16(oacc[2 * np][0], oacc[2 * np][1]), pack_bf16(oacc[2 * np][2], oacc[2 * np][3]),
                          pack_bf16(oacc[2 * np + 1][0], oacc[2 * np + 1][1]), pack_bf16(oacc[2 * np + 1][2], oacc[2 * np + 1][3]));
            }
            __syncwarp();
            unsigned char* og = reinterpret_cast<unsigned char*>(p.o) +
                                ((size_t)(bos + c * BT) * p.H + h) * (size_t)(DV * 2) + vb * 2;
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                int row = it * 16 + (lane >> 1), hf = lane & 1;
                if (row < valid) {
                    uint4 val = *reinterpret_cast<const uint4*>(stg + row * 32 + hf * 16);
                    *reinterpret_cast<uint4*>(og + (size_t)row * p.H * (DV * 2) + hf * 16) = val;
                }
            }
            __syncwarp();
        }

        // ---- S^T <- S^T diag(decay) + v_new^T kg ----
        {
            const float* dec = reinterpret_cast<const float*>(smem + s * L::STAGE_BYTES + L::DECAY);
#pragma unroll
            for (int jt = 0; jt < 16; ++jt) {
                float2 d2 = *reinterpret_cast<const float2*>(dec + 8 * jt + 2 * t);
                S[jt][0] *= d2.x; S[jt][1] *= d2.y; S[jt][2] *= d2.x; S[jt][3] *= d2.y;
            }
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
                for (int jp = 0; jp < 8; ++jp) {
                    uint32_t b0, b1, b2, b3;
                    int row = 16 * ks + (m & 1) * 8 + r, ch = 2 * jp + (m >> 1);
                    ldsm_x4_t(st + L::KG + row * 256 + ((ch ^ r) << 4), b0, b1, b2, b3);
                    mma_f16(S[2 * jp], va[ks], b0, b1);
                    mma_f16(S[2 * jp + 1], va[ks], b2, b3);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }

    float* final_dst = is_m ? p.m_out : p.ht;
    if (final_dst) {
        float* ht = final_dst + ((size_t)n * p.H + h) * DK * DV;
#pragma unroll
        for (int jt = 0; jt < 16; ++jt) {
            int k0 = 8 * jt + 2 * t;
            ht[(size_t)k0 * DV + vb + g] = S[jt][0];
            ht[(size_t)(k0 + 1) * DV + vb + g] = S[jt][1];
            ht[(size_t)k0 * DV + vb + g + 8] = S[jt][2];
            ht[(size_t)(k0 + 1) * DV + vb + g + 8] = S[jt][3];
        }
    }
}

}  // namespace kda

extern "C" int kda_fwd_scan_smem_bytes() { return kda::SCAN_SMEM; }

namespace {
// Launch with programmatic stream serialization: the grid may be scheduled while the previous kernel of the stream (the
// chunk-parallel stage) is still draining; every thread calls pdl_wait() before it reads anything.
template <typename Kernel>
cudaError_t launch_after_producer(Kernel kernel, dim3 grid, int threads, int smem, cudaStream_t stream, const kda::ScanParams& p) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}
}  // namespace

extern "C" int kda_launch_fwd_scan(const kda::ScanParams* p, cudaStream_t stream) {
    using namespace kda;
    if (p->N <= 0) return 0;
    dim3 grid(2, p->H, p->N);
    cudaError_t e;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const bool both_halves = 2LL * p->H * p->N > sms;      // more half-state CTAs than SMs: eight consumer warps per CTA
    using L2 = ScanLayout<false, 2>;
    if (p->vnew_out) {
        if (both_halves) {
            e = cudaFuncSetAttribute(kda_fwd_scan_kernel<true, false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, L2::SMEM);
            if (e != cudaSuccess) return (int)e;
            kda_fwd_scan_kernel<true, false, 2><<<dim3(1, p->H, p->N), (L2::CONSUMERS + 1) * 32, L2::SMEM, stream>>>(*p);
        } else {
            e = cudaFuncSetAttribute(kda_fwd_scan_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SCAN_SMEM);
            if (e != cudaSuccess) return (int)e;
            kda_fwd_scan_kernel<true, false><<<grid, SCAN_THREADS, SCAN_SMEM, stream>>>(*p);
        }
    } else {
        if (both_halves) {
            e = cudaFuncSetAttribute(kda_fwd_scan_kernel<false, false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, L2::SMEM);
            if (e != cudaSuccess) return (int)e;
            e = launch_after_producer(kda_fwd_scan_kernel<false, false, 2>, dim3(1, p->H, p->N), (L2::CONSUMERS + 1) * 32, L2::SMEM, stream, *p);
            if (e != cudaSuccess) return (int)e;
        } else {
            e = cudaFuncSetAttribute(kda_fwd_scan_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SCAN_SMEM);
            if (e != cudaSuccess) return (int)e;
            e = launch_after_producer(kda_fwd_scan_kernel<false, false>, grid, SCAN_THREADS, SCAN_SMEM, stream, *p);
            if (e != cudaSuccess) return (int)e;
        }
    }
    return (int)cudaGetLastError();
}

// Affine shard transitions of every (sequence, head): p->ht receives C, p->m_out receives M; p->o / p->h0 unused.
extern "C" int kda_launch_fwd_transition(const kda::ScanParams* p, cudaStream_t stream) {
    using namespace kda;
    if (p->N <= 0) return 0;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    ScanParams q = *p;
    q.group_major = 4LL * p->H * p->N > sms;     // see the index mapping at the top of the kernel
    const dim3 grid = q.group_major ? dim3(p->H, p->N, 4) : dim3(4, p->H, p->N);
    constexpr int smem = ScanLayout<true, 1>::SMEM;
    cudaError_t e = cudaFuncSetAttribute(kda_fwd_scan_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    kda_fwd_scan_kernel<false, true><<<grid, SCAN_THREADS, smem, stream>>>(q);
    return (int)cudaGetLastError();
}
