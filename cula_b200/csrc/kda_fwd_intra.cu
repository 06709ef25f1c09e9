// Chunk-parallel forward stage: one CTA per (chunk, head) fuses
//   gate activation + per-chunk cumulative sum (log2 domain), q/k L2 normalisation,
//   the gated 64x64 Gram matrices Aqk / L, Akk = (I + L)^-1, w = Akk (beta k 2^g), u = Akk (beta v),
//   kg = k 2^(g_last - g), qg = scale q 2^g,
// and writes the tile pack the state scan consumes (layout in kda_common.cuh).
//
// It replaces, in one launch, what the reference does with l2norm_fwd x2 (cula/kda/chunk.py:58-60),
// kda_gate_chunk_cumsum (cula/kda/chunk_fwd.py:69-78), chunk_kda_fwd_intra_cuda and
// recompute_w_u_cuda (csrc/api/kda_sm100.cu:22-120), so the fp32 gate, q-hat and k-hat never
// travel through HBM.
#include "kda_common.cuh"
#include "kda_params.h"

namespace kda {

constexpr int INTRA_THREADS = 256;

struct IntraSmem {
    float G[BT][DK];      // cumulative log2 gate; rows past the last real token repeat the last value
    float Q[BT][DK];      // q-hat (zero for padding rows)
    float Kh[BT][DK];     // k-hat (zero for padding rows)
    float L[BT][BT];      // strictly lower: beta_i * sum_d k_i k_j 2^(g_i-g_j)
    float P[BT][BT];      // lower incl. diagonal: scale * sum_d q_i k_j 2^(g_i-g_j)
    float A[BT][BT];      // (I + L)^-1
    float beta[BT];
    float half_total[DK];
};

__device__ __forceinline__ float load_gate_raw(const void* g, int g_fp32, size_t idx) {
    return g_fp32 ? reinterpret_cast<const float*>(g)[idx]
                  : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[idx]);
}

__device__ __forceinline__ float gate_activation(float graw, float alpha, float bias, int gate_mode, float lower_bound) {
    if (gate_mode == GATE_NONE) return graw;
    float x = graw + bias;
    if (gate_mode == GATE_LOWER_BOUND) return lower_bound / (1.f + __expf(-alpha * x));
    // softplus with the usual large-argument shortcut
    return -alpha * (x > 20.f ? x : log1pf(__expf(x)));
}

__global__ void __launch_bounds__(INTRA_THREADS, 1) kda_fwd_intra_kernel(const IntraParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    IntraSmem& s = *reinterpret_cast<IntraSmem*>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c = blockIdx.x / p.H, h = blockIdx.x - c * p.H;
    const ChunkInfo ci = chunk_info(c, p.cu_seqlens, p.chunk_indices, p.T);
    const size_t tok_stride = (size_t)p.H * DK;          // elements between consecutive tokens (K == V)
    const size_t base = (size_t)ci.row0 * tok_stride + (size_t)h * DK;
    unsigned char* tile = p.tiles + ((size_t)c * p.H + h) * TP_BYTES;

    // ---- 1. gate activation + cumulative sum down the 64 rows, two half-columns per channel ----
    {
        const int d = tid & 127, half = tid >> 7;
        const float alpha = p.gate_mode != GATE_NONE ? __expf(p.A_log[h]) : 0.f;
        const float bias = (p.gate_mode != GATE_NONE && p.dt_bias) ? p.dt_bias[h * DK + d] : 0.f;
        float run = 0.f;
#pragma unroll 4
        for (int r = 0; r < 32; ++r) {
            int row = half * 32 + r;
            float a = 0.f;
            if (row < ci.valid)
                a = gate_activation(load_gate_raw(p.g, p.g_fp32, base + (size_t)row * tok_stride + d), alpha, bias,
                                    p.gate_mode, p.lower_bound);
            run += a * RCP_LN2;
            s.G[row][d] = run;
        }
        if (half == 0) s.half_total[d] = run;
        __syncthreads();
        if (half == 1) {
            float t0 = s.half_total[d];
#pragma unroll 4
            for (int r = 32; r < 64; ++r) s.G[r][d] += t0;
        }
    }
    // ---- 2. L2 norms (a warp per row), beta ----
    {
        const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(p.q);
        const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(p.k);
        for (int r = 0; r < 8; ++r) {
            int row = warp * 8 + r;
            float qv[4] = {0, 0, 0, 0}, kv[4] = {0, 0, 0, 0};
            if (row < ci.valid) {
                uint2 qr = *reinterpret_cast<const uint2*>(qp + base + (size_t)row * tok_stride + lane * 4);
                uint2 kr = *reinterpret_cast<const uint2*>(kp + base + (size_t)row * tok_stride + lane * 4);
                float2 a = unpack_bf16(qr.x), b = unpack_bf16(qr.y);
                qv[0] = a.x; qv[1] = a.y; qv[2] = b.x; qv[3] = b.y;
                a = unpack_bf16(kr.x); b = unpack_bf16(kr.y);
                kv[0] = a.x; kv[1] = a.y; kv[2] = b.x; kv[3] = b.y;
            }
            float rq = 1.f, rk = 1.f;
            if (p.use_l2norm) {
                float sq = qv[0] * qv[0] + qv[1] * qv[1] + qv[2] * qv[2] + qv[3] * qv[3];
                float sk = kv[0] * kv[0] + kv[1] * kv[1] + kv[2] * kv[2] + kv[3] * kv[3];
#pragma unroll
                for (int o = 16; o; o >>= 1) {
                    sq += __shfl_xor_sync(0xffffffffu, sq, o);
                    sk += __shfl_xor_sync(0xffffffffu, sk, o);
                }
                rq = rsqrtf(sq + 1e-6f);
                rk = rsqrtf(sk + 1e-6f);
            }
            *reinterpret_cast<float4*>(&s.Q[row][lane * 4]) = make_float4(qv[0] * rq, qv[1] * rq, qv[2] * rq, qv[3] * rq);
            *reinterpret_cast<float4*>(&s.Kh[row][lane * 4]) = make_float4(kv[0] * rk, kv[1] * rk, kv[2] * rk, kv[3] * rk);
        }
        if (tid < BT) {
            float b = 0.f;
            if (tid < ci.valid) {
                size_t bi = (size_t)(ci.row0 + tid) * p.H + h;
                b = p.beta_fp32 ? reinterpret_cast<const float*>(p.beta)[bi]
                                : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.beta)[bi]);
            }
            s.beta[tid] = b;
        }
        for (int i = tid; i < BT * BT; i += INTRA_THREADS) {
            (&s.L[0][0])[i] = 0.f;
            (&s.P[0][0])[i] = 0.f;
        }
    }
    __syncthreads();

    // ---- 3. gated Gram matrices on the lower-triangular 4x4 blocks (136 of them); the other
    //         threads meanwhile emit kg, qg and the decay vector ----
    if (tid < 136) {
        int bi = (int)((sqrtf(8.f * tid + 1.f) - 1.f) * 0.5f);
        while ((bi + 1) * (bi + 2) / 2 <= tid) ++bi;
        while (bi * (bi + 1) / 2 > tid) --bi;
        const int bj = tid - bi * (bi + 1) / 2;
        float accP[4][4], accL[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) accP[a][b] = accL[a][b] = 0.f;
        for (int dd = 0; dd < DK; ++dd) {
            const int d = (dd + lane) & (DK - 1);      // rotate per lane: conflict-free column reads
            float qi[4], ki[4], gi[4], kj[4], gj[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                qi[a] = s.Q[4 * bi + a][d];
                ki[a] = s.Kh[4 * bi + a][d];
                gi[a] = s.G[4 * bi + a][d];
                kj[a] = s.Kh[4 * bj + a][d];
                gj[a] = s.G[4 * bj + a][d];
            }
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    float e = fast_exp2(fminf(gi[a] - gj[b], 0.f)) * kj[b];
                    accP[a][b] = fmaf(qi[a], e, accP[a][b]);
                    accL[a][b] = fmaf(ki[a], e, accL[a][b]);
                }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                int i = 4 * bi + a, j = 4 * bj + b;
                s.P[i][j] = (j <= i) ? p.scale * accP[a][b] : 0.f;
                s.L[i][j] = (j < i) ? s.beta[i] * accL[a][b] : 0.f;
            }
    } else {
        // kg / qg: one item = (row, 8 consecutive channels) -> one 16-byte store each
        for (int it = tid - 136; it < BT * 16; it += INTRA_THREADS - 136) {
            int row = it >> 4, ch = it & 15;
            uint32_t kgp[4], qgp[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int d = ch * 8 + 2 * e;
                float g0 = s.G[row][d], g1 = s.G[row][d + 1];
                float gl0 = s.G[BT - 1][d], gl1 = s.G[BT - 1][d + 1];
                kgp[e] = pack_f16(s.Kh[row][d] * fast_exp2(gl0 - g0), s.Kh[row][d + 1] * fast_exp2(gl1 - g1));
                qgp[e] = pack_f16(p.scale * s.Q[row][d] * fast_exp2(g0), p.scale * s.Q[row][d + 1] * fast_exp2(g1));
            }
            int off = swz256(row, ch * 8);
            *reinterpret_cast<uint4*>(tile + TP_KG + off) = make_uint4(kgp[0], kgp[1], kgp[2], kgp[3]);
            *reinterpret_cast<uint4*>(tile + TP_QG + off) = make_uint4(qgp[0], qgp[1], qgp[2], qgp[3]);
        }
        for (int d = tid - 136; d < DK; d += INTRA_THREADS - 136)
            reinterpret_cast<float*>(tile + TP_DECAY)[d] = fast_exp2(s.G[BT - 1][d]);
    }
    __syncthreads();

    // ---- 4. Akk = (I + L)^-1 by forward substitution, one column per thread (64 threads) ----
    if (tid < BT) {
        float x[BT];
#pragma unroll
        for (int i = 0; i < BT; ++i) {
            float acc = (i == tid) ? 1.f : 0.f;
#pragma unroll
            for (int j = 0; j < i; ++j) acc = fmaf(-s.L[i][j], x[j], acc);
            x[i] = acc;
        }
#pragma unroll
        for (int i = 0; i < BT; ++i) s.A[i][tid] = x[i];
    } else {
        // Aqk (fp16) into the pack
        for (int it = tid - BT; it < BT * 8; it += INTRA_THREADS - BT) {
            int row = it >> 3, ch = it & 7;
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) pk[e] = pack_f16(s.P[row][ch * 8 + 2 * e], s.P[row][ch * 8 + 2 * e + 1]);
            *reinterpret_cast<uint4*>(tile + TP_AQK + swz128(row, ch * 8)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
    }
    __syncthreads();

    // ---- 5. w = Akk X (threads 0..127, one key channel each), u = Akk Y (threads 128..255) ----
    {
        const int col = tid & 127, is_u = tid >> 7;
        float x[BT];
        if (is_u) {
            const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(p.v);
#pragma unroll
            for (int j = 0; j < BT; ++j)
                x[j] = (j < ci.valid) ? s.beta[j] * __bfloat162float(vp[base + (size_t)j * tok_stride + col]) : 0.f;
        } else {
#pragma unroll
            for (int j = 0; j < BT; ++j) x[j] = s.beta[j] * s.Kh[j][col] * fast_exp2(s.G[j][col]);
        }
        unsigned char* dst = is_u ? tile + (col < 64 ? TP_U0 : TP_U1) : tile + TP_W;
#pragma unroll
        for (int i = 0; i < BT; ++i) {
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j <= i; ++j) acc = fmaf(s.A[i][j], x[j], acc);
            if (is_u) *reinterpret_cast<__half*>(dst + swz128(i, col & 63)) = __float2half_rn(acc);
            else *reinterpret_cast<__half*>(dst + swz256(i, col)) = __float2half_rn(acc);
        }
    }
    // ---- 6. optional: Akk for the backward pass, fp32 row-major ----
    if (p.akk_out) {
        float* ao = p.akk_out + ((size_t)c * p.H + h) * BT * BT;
        for (int i = tid; i < BT * BT; i += INTRA_THREADS) ao[i] = (&s.A[0][0])[i];
    }
}

}  // namespace kda

extern "C" int kda_fwd_intra_smem_bytes() { return (int)sizeof(kda::IntraSmem); }

extern "C" int kda_launch_fwd_intra(const kda::IntraParams* p, int num_chunks, cudaStream_t stream) {
    using namespace kda;
    static_assert(sizeof(IntraSmem) <= 227 * 1024, "smem budget");
    if (num_chunks <= 0) return 0;
    cudaError_t e = cudaFuncSetAttribute(kda_fwd_intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(IntraSmem));
    if (e != cudaSuccess) return (int)e;
    kda_fwd_intra_kernel<<<num_chunks * p->H, INTRA_THREADS, sizeof(IntraSmem), stream>>>(*p);
    return (int)cudaGetLastError();
}
