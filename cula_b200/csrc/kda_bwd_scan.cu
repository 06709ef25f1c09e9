// Reverse state scan of the backward pass (mirror of kda_fwd_scan.cu).
//
// One CTA per (sequence, head, half of the value columns); four consumer warps each own 16 value columns of
// the fp32 state gradient dS^T (16 x 128 per warp) in mma.sync accumulator registers and walk the chunks
// from last to first:
//     dVn^T  = dS'^T Kg^T + dO^T Aqk                 (gradient w.r.t. v_new; stored for the chunk-parallel stage)
//     dS^T  <- dS'^T diag(decay) + dO^T Qg - dVn^T W  (gradient w.r.t. the state entering the chunk)
// A fifth warp streams the forward tile packs (W, QG, KG, AQK, DECAY) and the dO rows of the chunk through a
// 3-stage shared-memory ring with bulk copies on mbarriers.
//
// Replaces chunk_gated_delta_rule_bwd_dhu (flash-linear-attention, fla/ops/common/chunk_delta_h.py:316-718, called
// at cula/kda/chunk_bwd.py:541-555) and the dv half of chunk_kda_bwd_kernel_dAv (cula/kda/chunk_bwd.py:63-125).
//
// Range: every gradient-like operand (dO, dht, dS', dVn) is carried in units of a power-of-two scale s chosen
// from max|dO|, max|dht| (kda_grad_scale_kernel), so fp16 MMA operands neither overflow nor go subnormal.
#include "kda_common.cuh"
#include "kda_params.h"

namespace kda {

constexpr int BS_STAGES = 3;
constexpr int BS_DO_ROW = 144;                               // padded dO row (64 bf16 + 16 B): conflict-free ldmatrix
constexpr int BS_DO_BYTES = BT * BS_DO_ROW;                  // 9216
constexpr int BS_STAGE_BYTES = TP_HEAD_BYTES + BS_DO_BYTES;  // 67072
constexpr int BS_STG_BYTES = 2048;                           // per-warp staging for the dVn store
constexpr int BS_CONSUMERS = 4;
constexpr int BS_THREADS = (BS_CONSUMERS + 1) * 32;
constexpr int BS_SMEM = BS_STAGES * BS_STAGE_BYTES + BS_CONSUMERS * BS_STG_BYTES + 64;
constexpr int BS_DO = TP_HEAD_BYTES;

// s = 2^k with max(|dO|, |dht|) * s in [4, 8); written as {s, 1/s}. amax_bits holds the running maximum.
__global__ void kda_grad_amax_kernel(const __nv_bfloat16* d_o, size_t n_do, const float* dht, size_t n_dht,
                                     unsigned int* amax_bits) {
    float m = 0.f;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (size_t)gridDim.x * blockDim.x;
    // 16-byte loads over the bulk (the tensors come 16-byte aligned from the C ABI), scalar loads over the tail
    const uint4* do4 = reinterpret_cast<const uint4*>(d_o);
    for (size_t i = tid; i < n_do / 8; i += nthr) {
        const uint4 v = do4[i];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = unpack_bf16(w[e]);
            m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
    }
    for (size_t i = (n_do / 8) * 8 + tid; i < n_do; i += nthr) m = fmaxf(m, fabsf(__bfloat162float(d_o[i])));
    const float4* h4 = reinterpret_cast<const float4*>(dht);
    for (size_t i = tid; i < n_dht / 4; i += nthr) {
        const float4 v = h4[i];
        m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    for (size_t i = (n_dht / 4) * 4 + tid; i < n_dht; i += nthr) m = fmaxf(m, fabsf(dht[i]));
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m > 0.f && m < INFINITY) atomicMax(amax_bits, __float_as_uint(m));
}
__global__ void kda_grad_scale_kernel(const unsigned int* amax_bits, float* gscale) {
    const float m = __uint_as_float(*amax_bits);
    int e = ((__float_as_int(m) >> 23) & 0xff) - 127;      // floor(log2 m); m == 0 gives -127
    int shift = (m > 0.f) ? 2 - e : 0;
    shift = max(-120, min(120, shift));
    gscale[0] = __int_as_float((shift + 127) << 23);
    gscale[1] = __int_as_float((127 - shift) << 23);
}

__global__ void __launch_bounds__(BS_THREADS, 1) kda_bwd_scan_kernel(const BwdScanParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + BS_STAGES * BS_STAGE_BYTES + BS_CONSUMERS * BS_STG_BYTES);
    uint64_t* empty = full + BS_STAGES;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int vh = blockIdx.x, h = blockIdx.y;
    const int n = p.seq_order ? p.seq_order[blockIdx.z] : blockIdx.z;
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
        for (int s = 0; s < BS_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], BS_CONSUMERS);
        }
        fence_mbar_init();
    }
    __syncthreads();

    if (warp == BS_CONSUMERS) {
        // ------------------------------- producer warp (all lanes copy dO rows) -------------------------------
        const __nv_bfloat16* dop = reinterpret_cast<const __nv_bfloat16*>(p.d_o);
        for (int it = 0; it < nchunks; ++it) {
            const int c = nchunks - 1 - it;
            const int s = it % BS_STAGES, use = it / BS_STAGES;
            const int valid = min(BT, len - c * BT);
            bool ok = true;
            if (lane == 0 && use > 0) ok = mbar_wait(&empty[s], (use - 1) & 1);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0) atomicExch(p.status, STATUS_WAIT_TIMEOUT);
                break;
            }
            unsigned char* dst = smem + s * BS_STAGE_BYTES;
            // rows past the end of the sequence are never copied: clear them so stale bytes cannot inject NaNs
            for (int i = lane; i < (BT - valid) * 8; i += 32)
                *reinterpret_cast<uint4*>(dst + BS_DO + (valid + (i >> 3)) * BS_DO_ROW + (i & 7) * 16) = make_uint4(0, 0, 0, 0);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_expect_tx(&full[s], TP_HEAD_BYTES + valid * 128);
                bulk_g2s(dst, p.tiles + ((size_t)(chunk0 + c) * p.H + h) * TP_BYTES, TP_HEAD_BYTES, &full[s]);
            }
            __syncwarp();
            for (int row = lane; row < valid; row += 32)
                bulk_g2s(dst + BS_DO + row * BS_DO_ROW,
                         dop + ((size_t)(bos + c * BT + row) * p.H + h) * DV + vh * 64, 128, &full[s]);
        }
        return;
    }

    // ---------------------------------- consumer warps ----------------------------------
    const int g = lane >> 2, t = lane & 3;
    const int m = lane >> 3, r = lane & 7;
    const int vb = vh * 64 + warp * 16;
    unsigned char* stg = smem + BS_STAGES * BS_STAGE_BYTES + warp * BS_STG_BYTES;
    const uint32_t stg_u32 = smem_u32(stg);
    const float gs = p.gscale[0], gs_inv = p.gscale[1];

    float S[16][4];     // dS^T tile: rows v (g, g+8), cols k = 8*jt + 2t, +1; units of gs
    if (p.dht) {
        const float* d0 = p.dht + ((size_t)n * p.H + h) * DK * DV;
#pragma unroll
        for (int jt = 0; jt < 16; ++jt) {
            int k0 = 8 * jt + 2 * t;
            S[jt][0] = gs * d0[(size_t)k0 * DV + vb + g];
            S[jt][1] = gs * d0[(size_t)(k0 + 1) * DV + vb + g];
            S[jt][2] = gs * d0[(size_t)k0 * DV + vb + g + 8];
            S[jt][3] = gs * d0[(size_t)(k0 + 1) * DV + vb + g + 8];
        }
    } else {
#pragma unroll
        for (int jt = 0; jt < 16; ++jt) S[jt][0] = S[jt][1] = S[jt][2] = S[jt][3] = 0.f;
    }
    uint32_t x256[4];
#pragma unroll
    for (int kp = 0; kp < 4; ++kp) x256[kp] = (uint32_t)(((4 * kp + m) ^ r) << 4);

    for (int it = 0; it < nchunks; ++it) {
        const int c = nchunks - 1 - it;
        const int s = it % BS_STAGES;
        if (!mbar_wait(&full[s], (it / BS_STAGES) & 1)) {
            atomicExch(p.status, STATUS_WAIT_TIMEOUT);
            return;
        }
        const uint32_t st = smem_u32(smem + s * BS_STAGE_BYTES);
        const size_t tile_idx = (size_t)(chunk0 + c) * p.H + h;

        // ---- dS' (gradient w.r.t. the state leaving this chunk) to HBM, fp32 [128 k][128 v] ----
        if (p.ds_out) {
            float* dsg = p.ds_out + tile_idx * (size_t)(DK * DV);
#pragma unroll
            for (int jt = 0; jt < 16; ++jt) {
                int k0 = 8 * jt + 2 * t;
                dsg[(size_t)k0 * DV + vb + g] = S[jt][0];
                dsg[(size_t)(k0 + 1) * DV + vb + g] = S[jt][1];
                dsg[(size_t)k0 * DV + vb + g + 8] = S[jt][2];
                dsg[(size_t)(k0 + 1) * DV + vb + g + 8] = S[jt][3];
            }
        }
        // ---- dS' as fp16 A fragments with a per-warp power-of-two scale ----
        float smax = 0.f;
#pragma unroll
        for (int jt = 0; jt < 16; ++jt)
            smax = fmaxf(smax, fmaxf(fmaxf(fabsf(S[jt][0]), fabsf(S[jt][1])), fmaxf(fabsf(S[jt][2]), fabsf(S[jt][3]))));
#pragma unroll
        for (int o = 16; o; o >>= 1) smax = fmaxf(smax, __shfl_xor_sync(0xffffffffu, smax, o));
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
        // ---- dO^T as fp16 A fragments (units of gs): 4 k-steps over the 64 tokens ----
        uint32_t doa[4][4];
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t r0, r1, r2, r3;
            ldsm_x4_t(st + BS_DO + (16 * ks + (m >> 1) * 8 + r) * BS_DO_ROW + (2 * warp + (m & 1)) * 16, r0, r1, r2, r3);
            float2 f;
            f = unpack_bf16(r0); doa[ks][0] = pack_f16(gs * f.x, gs * f.y);
            f = unpack_bf16(r1); doa[ks][1] = pack_f16(gs * f.x, gs * f.y);
            f = unpack_bf16(r2); doa[ks][2] = pack_f16(gs * f.x, gs * f.y);
            f = unpack_bf16(r3); doa[ks][3] = pack_f16(gs * f.x, gs * f.y);
        }
        // ---- dVn^T = dS'^T Kg^T + dO^T Aqk : [16 v] x [64 tokens] ----
        float acc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
        for (int kp = 0; kp < 4; ++kp) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(st + TP_KG + (8 * nt + r) * 256 + x256[kp], b0, b1, b2, b3);
                mma_f16(acc[nt], sa[2 * kp], b0, b1);
                mma_f16(acc[nt], sa[2 * kp + 1], b2, b3);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            acc[nt][0] *= s_down; acc[nt][1] *= s_down; acc[nt][2] *= s_down; acc[nt][3] *= s_down;
        }
        // B[k = token j][n = token i] = Aqk[j][i]: rows j, 16-byte groups along i -> transposed ldmatrix
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                if (16 * np <= 16 * ks + 15) {          // Aqk[j][i] = 0 for i > j
                    uint32_t b0, b1, b2, b3;
                    const int row = 16 * ks + (m & 1) * 8 + r, ch = 2 * np + (m >> 1);
                    ldsm_x4_t(st + TP_AQK + row * 128 + ((ch ^ r) << 4), b0, b1, b2, b3);
                    mma_f16(acc[2 * np], doa[ks], b0, b1);
                    mma_f16(acc[2 * np + 1], doa[ks], b2, b3);
                }
            }
        }
        uint32_t va[4][4];   // dVn^T as fp16 A fragments
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            va[ks][0] = pack_f16(acc[2 * ks][0], acc[2 * ks][1]);
            va[ks][1] = pack_f16(acc[2 * ks][2], acc[2 * ks][3]);
            va[ks][2] = pack_f16(acc[2 * ks + 1][0], acc[2 * ks + 1][1]);
            va[ks][3] = pack_f16(acc[2 * ks + 1][2], acc[2 * ks + 1][3]);
        }
        if (p.dvn_out) {   // dVn, fp16 [64 tokens][128 v]
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                int trow = 8 * (2 * ks + (m >> 1)) + r;
                stsm_x4_t(stg_u32 + trow * 32 + (m & 1) * 16, va[ks][0], va[ks][1], va[ks][2], va[ks][3]);
            }
            __syncwarp();
            unsigned char* vg = reinterpret_cast<unsigned char*>(p.dvn_out) + tile_idx * (size_t)(BT * DV * 2);
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
                int row = i4 * 16 + (lane >> 1), hf = lane & 1;
                uint4 val = *reinterpret_cast<const uint4*>(stg + row * 32 + hf * 16);
                *reinterpret_cast<uint4*>(vg + (size_t)row * 256 + vb * 2 + hf * 16) = val;
            }
            __syncwarp();
        }
        // ---- dS^T <- dS'^T diag(decay) + dO^T Qg - dVn^T W ----
        {
            const float* dec = reinterpret_cast<const float*>(smem + s * BS_STAGE_BYTES + TP_DECAY);
#pragma unroll
            for (int jt = 0; jt < 16; ++jt) {
                float2 d2 = *reinterpret_cast<const float2*>(dec + 8 * jt + 2 * t);
                S[jt][0] *= d2.x; S[jt][1] *= d2.y; S[jt][2] *= d2.x; S[jt][3] *= d2.y;
            }
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                uint32_t vneg[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) vneg[e] = va[ks][e] ^ 0x80008000u;
#pragma unroll
                for (int jp = 0; jp < 8; ++jp) {
                    uint32_t b0, b1, b2, b3;
                    const int row = 16 * ks + (m & 1) * 8 + r, ch = 2 * jp + (m >> 1);
                    const uint32_t off = row * 256 + ((ch ^ r) << 4);
                    ldsm_x4_t(st + TP_QG + off, b0, b1, b2, b3);
                    mma_f16(S[2 * jp], doa[ks], b0, b1);
                    mma_f16(S[2 * jp + 1], doa[ks], b2, b3);
                    ldsm_x4_t(st + TP_W + off, b0, b1, b2, b3);
                    mma_f16(S[2 * jp], vneg, b0, b1);
                    mma_f16(S[2 * jp + 1], vneg, b2, b3);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }

    if (p.dh0) {
        float* d0 = p.dh0 + ((size_t)n * p.H + h) * DK * DV;
#pragma unroll
        for (int jt = 0; jt < 16; ++jt) {
            int k0 = 8 * jt + 2 * t;
            d0[(size_t)k0 * DV + vb + g] = gs_inv * S[jt][0];
            d0[(size_t)(k0 + 1) * DV + vb + g] = gs_inv * S[jt][1];
            d0[(size_t)k0 * DV + vb + g + 8] = gs_inv * S[jt][2];
            d0[(size_t)(k0 + 1) * DV + vb + g + 8] = gs_inv * S[jt][3];
        }
    }
}

}  // namespace kda

extern "C" int kda_launch_grad_scale(const void* d_o, size_t n_do, const float* dht, size_t n_dht, unsigned int* amax_bits,
                                     float* gscale, cudaStream_t stream) {
    using namespace kda;
    cudaError_t e = cudaMemsetAsync(amax_bits, 0, sizeof(unsigned int), stream);
    if (e != cudaSuccess) return (int)e;
    kda_grad_amax_kernel<<<1184, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(d_o), n_do, dht, dht ? n_dht : 0,
                                                  amax_bits);
    kda_grad_scale_kernel<<<1, 1, 0, stream>>>(amax_bits, gscale);
    return (int)cudaGetLastError();
}

extern "C" int kda_launch_bwd_scan(const kda::BwdScanParams* p, cudaStream_t stream) {
    using namespace kda;
    if (p->N <= 0) return 0;
    dim3 grid(2, p->H, p->N);
    cudaError_t e = cudaFuncSetAttribute(kda_bwd_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BS_SMEM);
    if (e != cudaSuccess) return (int)e;
    kda_bwd_scan_kernel<<<grid, BS_THREADS, BS_SMEM, stream>>>(*p);
    return (int)cudaGetLastError();
}
