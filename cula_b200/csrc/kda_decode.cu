// KDA decode: one token per sequence against a pool of fp32 states, updated in place.
//     gate  = exp(-exp(A_log[hv]) * softplus(a + dt_bias[hv, :]))            [K]
//     v_new = sigmoid(b) * (v - S^T (gate * k_hat))                           [V]
//     S    <- diag(gate) S + k_hat v_new^T                                    [K x V]
//     o     = S^T (scale * q_hat)                                             [V]
// per (sequence n, value head hv); q/k head = hv / (HV / H) (grouped heads). Semantics of kda_decode /
// fused_sigmoid_gating_delta_rule_update (cula/ops/kda_decode.py:1794-2096) and of the reference's torch
// restatement (tests/test_kda_decode.py:42-104); a negative state index skips the sequence: no state access, as in
// the reference kernel (cula/ops/kda_decode.py:11-13), and a zero output row (the reference leaves it unwritten).
//
// The step is pure HBM streaming: 64 KB of state read and 64 KB written per (n, hv) against a few hundred bytes
// of vectors, so the kernel is organised around coalesced 16-byte accesses with many rows in flight:
//   layout "vk" (pool, HV, V, K), the reference's default: a warp walks its value rows 8 at a time (8 x 128
//     floats in registers, lane = 4 consecutive k, the next 8 rows already in flight), both contractions are
//     4 FMAs + a warp reduction per row;
//   layout "kv" (pool, HV, K, V): a CTA owns a 32-column value slice; a warp holds 32 key rows (8 lanes x
//     float4 per row), the contractions reduce over lanes with equal column group and across the 4 warps
//     through shared memory.
// Work items = N * HV * slices (K = 128; V any multiple of 32; slices divides V / 32 and is chosen on the host: 1
// when there are enough states to fill the GPU, more for small batches); four persistent CTAs of 128 threads
// per SM walk them.
#include "kda_common.cuh"

namespace kda {

struct DecodeParams {
    const void* q;        // [N, H, 128] bf16
    const void* k;        // [N, H, 128] bf16
    const void* v;        // [N, HV, V] bf16 (V a multiple of 32)
    const void* a;        // [N, HV, 128] bf16 or fp32 (raw gate input)
    const void* b;        // [N, HV] bf16 or fp32 (raw beta input)
    const float* A_log;   // [HV]
    const float* dt_bias; // [HV, 128] or nullptr
    float* state;         // [pool, HV, V, 128] (vk) or [pool, HV, 128, V] (kv) fp32, updated in place
    const int* indices;   // [N] pool slot of every sequence, or nullptr (slot = n)
    void* o;              // [N, HV, V] bf16
    int N, H, HV, V, pool, slices;   // slices: CTAs per state, each owning V / slices value rows (vk) or columns (kv)
    int a_fp32, b_fp32, use_l2norm, state_kv;
    float scale, softplus_beta, softplus_threshold;
    int* status;
};

constexpr int DEC_THREADS = 128;

__device__ __forceinline__ float dec_softplus(float x, float beta, float threshold) {
    const float bx = beta * x;
    return bx > threshold ? x : log1pf(__expf(bx)) / beta;      // torch.nn.functional.softplus(beta, threshold)
}
__device__ __forceinline__ float dec_load(const void* p, int is_fp32, size_t i) {
    return is_fp32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// The per-key vectors of one (n, hv) for the 4 keys k0..k0+3 of a lane that covers the key axis with 32 lanes:
// gate, k_hat, scale * q_hat. The L2 norms are warp reductions over the 128 keys.
__device__ __forceinline__ void dec_key_vectors(const DecodeParams& p, int n, int hv, int hq, int k0, float (&gate)[4], float (&kh)[4],
                                                float (&qs)[4]) {
    const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(p.q) + ((size_t)n * p.H + hq) * DK + k0;
    const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(p.k) + ((size_t)n * p.H + hq) * DK + k0;
    const uint2 qr = *reinterpret_cast<const uint2*>(qp), kr = *reinterpret_cast<const uint2*>(kp);
    float2 f;
    f = unpack_bf16(qr.x); qs[0] = f.x; qs[1] = f.y;
    f = unpack_bf16(qr.y); qs[2] = f.x; qs[3] = f.y;
    f = unpack_bf16(kr.x); kh[0] = f.x; kh[1] = f.y;
    f = unpack_bf16(kr.y); kh[2] = f.x; kh[3] = f.y;
    float rq = p.scale, rk = 1.f;
    if (p.use_l2norm) {
        float sq = qs[0] * qs[0] + qs[1] * qs[1] + qs[2] * qs[2] + qs[3] * qs[3];
        float sk = kh[0] * kh[0] + kh[1] * kh[1] + kh[2] * kh[2] + kh[3] * kh[3];
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
            sk += __shfl_xor_sync(0xffffffffu, sk, o);
        }
        rq = p.scale * rsqrtf(sq + 1e-6f);
        rk = rsqrtf(sk + 1e-6f);
    }
    const float alpha = __expf(p.A_log[hv]);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        qs[e] *= rq;
        kh[e] *= rk;
        const float x = dec_load(p.a, p.a_fp32, ((size_t)n * p.HV + hv) * DK + k0 + e) + (p.dt_bias ? p.dt_bias[hv * DK + k0 + e] : 0.f);
        gate[e] = __expf(-alpha * dec_softplus(x, p.softplus_beta, p.softplus_threshold));
    }
}

// One work item = one slice of one (sequence, value head) state.
__device__ __forceinline__ void dec_item(const DecodeParams& p, const int item, float (*red)[4][32], float* s_gate, float* s_kh,
                                         float* s_qs) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int slice = item % p.slices, nh = item / p.slices;
    const int per_cta = p.V / p.slices;                     // value rows (vk) or columns (kv) of this CTA, a multiple of 32
    const int n = nh / p.HV, hv = nh - n * p.HV;
    const int hq = hv / (p.HV / p.H);
    const int slot = p.indices ? p.indices[n] : n;
    if (slot < 0) {                                         // padded sequence: no state access; its output row is zeroed
        __nv_bfloat16* oz = reinterpret_cast<__nv_bfloat16*>(p.o) + ((size_t)n * p.HV + hv) * p.V + slice * per_cta;
        for (int i = tid; i < per_cta; i += DEC_THREADS) oz[i] = __float2bfloat16_rn(0.f);
        return;
    }
    if (slot >= p.pool) {                                   // caller error: report, touch nothing
        if (tid == 0) atomicExch(p.status, STATUS_BAD_INDEX);
        return;
    }
    float* S = p.state + ((size_t)slot * p.HV + hv) * (size_t)DK * p.V;
    const float beta = 1.f / (1.f + __expf(-dec_load(p.b, p.b_fp32, (size_t)n * p.HV + hv)));
    const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(p.v) + ((size_t)n * p.HV + hv) * p.V;
    __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.o) + ((size_t)n * p.HV + hv) * p.V;

    if (!p.state_kv) {
        // ---- (V, K) rows: the warp owns per_cta / 4 value rows and walks them 8 at a time, the next 8 already in
        //      flight while the current 8 are updated; the lane owns keys 4*lane .. 4*lane+3 ----
        const int rows_warp = per_cta >> 2, nb = rows_warp >> 3;
        const int vbase = slice * per_cta + warp * rows_warp, k0 = 4 * lane;
        float4 row[8], nxt[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) row[i] = __ldcs(reinterpret_cast<const float4*>(S + (size_t)(vbase + i) * DK + k0));
        float gate[4], kh[4], qs[4];
        dec_key_vectors(p, n, hv, hq, k0, gate, kh, qs);
        float gk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) gk[e] = gate[e] * kh[e];
        for (int bi = 0; bi < nb; ++bi) {
            const int v0 = vbase + 8 * bi;
            if (bi + 1 < nb) {
#pragma unroll
                for (int i = 0; i < 8; ++i) nxt[i] = __ldcs(reinterpret_cast<const float4*>(S + (size_t)(v0 + 8 + i) * DK + k0));
            }
            float hk[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) hk[i] = row[i].x * gk[0] + row[i].y * gk[1] + row[i].z * gk[2] + row[i].w * gk[3];
#pragma unroll
            for (int o = 16; o; o >>= 1)
#pragma unroll
                for (int i = 0; i < 8; ++i) hk[i] += __shfl_xor_sync(0xffffffffu, hk[i], o);
            float ov[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float vn = beta * (__bfloat162float(vp[v0 + i]) - hk[i]);
                row[i].x = fmaf(gate[0], row[i].x, vn * kh[0]);
                row[i].y = fmaf(gate[1], row[i].y, vn * kh[1]);
                row[i].z = fmaf(gate[2], row[i].z, vn * kh[2]);
                row[i].w = fmaf(gate[3], row[i].w, vn * kh[3]);
                __stcs(reinterpret_cast<float4*>(S + (size_t)(v0 + i) * DK + k0), row[i]);
                ov[i] = row[i].x * qs[0] + row[i].y * qs[1] + row[i].z * qs[2] + row[i].w * qs[3];
            }
#pragma unroll
            for (int o = 16; o; o >>= 1)
#pragma unroll
                for (int i = 0; i < 8; ++i) ov[i] += __shfl_xor_sync(0xffffffffu, ov[i], o);
            if (lane < 8) {
                float mine = ov[0];
#pragma unroll
                for (int i = 1; i < 8; ++i) mine = (lane == i) ? ov[i] : mine;
                op[v0 + lane] = __float2bfloat16_rn(mine);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) row[i] = nxt[i];
        }
        return;
    }

    // ---- (K, V) rows: the CTA walks its value columns 32 at a time; warp w owns key rows 32w .. 32w+31, lane (rg, cg):
    //      row group rg = lane / 8 (rows rg, rg+4, ..., rg+28 of the warp's 32), column group cg = lane % 8 ----
    {
        float gate[4], kh[4], qs[4];
        dec_key_vectors(p, n, hv, hq, 4 * lane, gate, kh, qs);       // every warp computes the same 128 values
        if (warp == 0) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s_gate[4 * lane + e] = gate[e];
                s_kh[4 * lane + e] = kh[e];
                s_qs[4 * lane + e] = qs[e];
            }
        }
    }
    const int rg = lane >> 3, cg = lane & 7;
    for (int c0 = slice * per_cta; c0 < (slice + 1) * per_cta; c0 += 32) {
    float4 row[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
        row[i] = __ldcs(reinterpret_cast<const float4*>(S + (size_t)(32 * warp + rg + 4 * i) * p.V + c0 + 4 * cg));
    __syncthreads();
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int kk = 32 * warp + rg + 4 * i;
        const float w = s_gate[kk] * s_kh[kk];
        acc.x = fmaf(row[i].x, w, acc.x); acc.y = fmaf(row[i].y, w, acc.y);
        acc.z = fmaf(row[i].z, w, acc.z); acc.w = fmaf(row[i].w, w, acc.w);
    }
#pragma unroll
    for (int o = 8; o < 32; o <<= 1) {
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o); acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o); acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
    }
    if (rg == 0) *reinterpret_cast<float4*>(&red[0][warp][4 * cg]) = acc;
    __syncthreads();
    float vn[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int c = 4 * cg + e;
        const float hk = (red[0][0][c] + red[0][1][c]) + (red[0][2][c] + red[0][3][c]);
        vn[e] = beta * (__bfloat162float(vp[c0 + c]) - hk);
    }
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int kk = 32 * warp + rg + 4 * i;
        const float gt = s_gate[kk], kh = s_kh[kk], qv = s_qs[kk];
        row[i].x = fmaf(gt, row[i].x, kh * vn[0]); row[i].y = fmaf(gt, row[i].y, kh * vn[1]);
        row[i].z = fmaf(gt, row[i].z, kh * vn[2]); row[i].w = fmaf(gt, row[i].w, kh * vn[3]);
        __stcs(reinterpret_cast<float4*>(S + (size_t)kk * p.V + c0 + 4 * cg), row[i]);
        acc.x = fmaf(row[i].x, qv, acc.x); acc.y = fmaf(row[i].y, qv, acc.y);
        acc.z = fmaf(row[i].z, qv, acc.z); acc.w = fmaf(row[i].w, qv, acc.w);
    }
#pragma unroll
    for (int o = 8; o < 32; o <<= 1) {
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o); acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o); acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
    }
    if (rg == 0) *reinterpret_cast<float4*>(&red[1][warp][4 * cg]) = acc;
    __syncthreads();
    if (tid < 32) op[c0 + tid] = __float2bfloat16_rn((red[1][0][tid] + red[1][1][tid]) + (red[1][2][tid] + red[1][3][tid]));
    }   // column chunks (the barriers above also order the reuse of `red`)
}

// Persistent: a few CTAs per SM walk the work items, so the short items do not pay a CTA launch each.
__global__ void __launch_bounds__(DEC_THREADS, 4) kda_decode_kernel(const DecodeParams p, const int items) {
    __shared__ float red[2][4][32];
    __shared__ float s_gate[DK], s_kh[DK], s_qs[DK];
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        dec_item(p, item, red, s_gate, s_kh, s_qs);
        if (p.state_kv) __syncthreads();                    // the shared vectors are rewritten by the next item
    }
}

}  // namespace kda

extern "C" int kda_launch_decode(const void* q, const void* k, const void* v, const void* a, int a_fp32, const void* b, int b_fp32,
                                 const float* A_log, const float* dt_bias, float* state, const int* indices, void* o,
                                 int N, int H, int HV, int V, int pool, float scale, int use_l2norm, float softplus_beta,
                                 float softplus_threshold, int state_kv, int* status, cudaStream_t stream) {
    using namespace kda;
    if (N <= 0) return 0;
    DecodeParams p{};
    p.q = q; p.k = k; p.v = v; p.a = a; p.b = b; p.A_log = A_log; p.dt_bias = dt_bias; p.state = state; p.indices = indices;
    p.o = o; p.N = N; p.H = H; p.HV = HV; p.V = V; p.pool = pool; p.a_fp32 = a_fp32; p.b_fp32 = b_fp32; p.use_l2norm = use_l2norm;
    p.state_kv = state_kv; p.scale = scale; p.softplus_beta = softplus_beta; p.softplus_threshold = softplus_threshold;
    p.status = status;
    // enough CTAs to fill the machine several times over, else as few (= as much work per CTA) as possible
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int slices = 1;
    while (slices < V / 32 && (long long)N * HV * slices < 8LL * sms && (V / 32) % (2 * slices) == 0) slices *= 2;
    p.slices = slices;
    const long long items = (long long)N * HV * slices;
    if (items > 0x7fffffffLL) return -1;
    const long long resident = 4LL * sms;                   // launch bounds keep four 128-thread CTAs resident per SM
    kda_decode_kernel<<<(int)(items < resident ? items : resident), DEC_THREADS, 0, stream>>>(p, (int)items);
    return (int)cudaGetLastError();
}
