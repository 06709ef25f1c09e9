// Layer-side elementwise operators that sit next to chunk_kda in a Kimi-Linear block, as stand-alone kernels:
//   kda_gate fwd / bwd   : a = -exp(A_log[h]) softplus(g + dt_bias[h,:])           (softplus form)
//                          a = lower_bound sigmoid(exp(A_log[h]) (g + dt_bias[h,:]))  (lower-bound form)
//   beta_sigmoid fwd/bwd : y = sigmoid(x) in fp32
// They replace flash-linear-attention's fused_kda_gate / fused_beta_sigmoid (fla/ops/kda/gate.py:282-345, 348-432),
// which the reference's callers use when the gate is not computed inside chunk_kda. Pure streaming work: every element
// is read once and written once; the two parameter gradients are block-reduced and finished with atomics.
#include "kda_common.cuh"
#include "kda_params.h"

namespace kda {

constexpr int GATE_THREADS = 256;


__device__ __forceinline__ void load8(const void* p, int fp32, size_t idx, float (&v)[8]) {
    if (fp32) {
        const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + idx);
        const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + idx + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 a = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + idx);
        float2 f;
        f = unpack_bf16(a.x); v[0] = f.x; v[1] = f.y;
        f = unpack_bf16(a.y); v[2] = f.x; v[3] = f.y;
        f = unpack_bf16(a.z); v[4] = f.x; v[5] = f.y;
        f = unpack_bf16(a.w); v[6] = f.x; v[7] = f.y;
    }
}
__device__ __forceinline__ void store8(void* p, int fp32, size_t idx, const float (&v)[8]) {
    if (fp32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + idx) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + idx + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p) + idx) =
            make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
    }
}
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// grid.x covers the H*K/8 channel groups (a thread keeps its 8 channels for the whole launch, so the bias and the
// head's exp(A_log) are loaded once), grid.y strides over the tokens.
template <bool BWD>
__global__ void __launch_bounds__(GATE_THREADS) kda_gate_kernel(const GateArgs a) {
    __shared__ float sDA[66];     // A_log gradient of the heads this block touches: at most 256 * 8 / K + 1, K >= 32
    const int HK = a.H * a.K, groups = HK / 8;
    const int grp = blockIdx.x * GATE_THREADS + threadIdx.x;
    const bool active = grp < groups;
    const int ch = active ? 8 * grp : 0, h = ch / a.K;
    const int h_lo = (blockIdx.x * GATE_THREADS * 8) / a.K;       // first head of this block
    if (BWD) {
        for (int i = threadIdx.x; i < 66; i += GATE_THREADS) sDA[i] = 0.f;
        __syncthreads();
    }
    const float alpha = __expf(a.A_log[h]);
    float bias[8], dbias[8], dA = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        bias[e] = (a.dt_bias && active) ? a.dt_bias[ch + e] : 0.f;
        dbias[e] = 0.f;
    }
    if (active) {
        // rows are taken four at a time and all their loads are issued before the first is used: a thread has only a
        // handful of rows, and one load per dependent step would make each of them pay a full memory latency
        constexpr int NB = 4;
        for (long long mb = blockIdx.y; mb < a.M; mb += (long long)NB * gridDim.y) {
            float gv[NB][8], dy[NB][8];
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const long long m = min(mb + (long long)i * gridDim.y, a.M - 1);      // clamped: the surplus rows are not used
                const size_t idx = (size_t)m * HK + ch;
                load8(a.g, a.g_fp32, idx, gv[i]);
                if (BWD) load8(a.dy, a.dy_fp32, idx, dy[i]);
            }
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const long long m = mb + (long long)i * gridDim.y;
                if (m >= a.M) break;
                const size_t idx = (size_t)m * HK + ch;
                float o[8];
                if (!BWD) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float x = gv[i][e] + bias[e];
                        o[e] = a.use_lower_bound ? a.lower_bound * __fdividef(1.f, 1.f + __expf(-alpha * x)) : -alpha * softplus_f(x);
                    }
                    store8(a.out, a.out_fp32, idx, o);
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float x = gv[i][e] + bias[e];
                        float v;
                        if (a.use_lower_bound) {
                            const float sg = __fdividef(1.f, 1.f + __expf(-alpha * x));
                            v = dy[i][e] * a.lower_bound * sg * (1.f - sg) * alpha;      // d/dx of lb sigmoid(alpha x)
                            dA = fmaf(v, x, dA);                                         // d/dA_log = d/d(alpha) * alpha
                        } else {
                            v = -dy[i][e] * alpha * __fdividef(1.f, 1.f + __expf(-x));
                            dA = fmaf(dy[i][e], -alpha * softplus_f(x), dA);
                        }
                        dbias[e] += v;
                        o[e] = v;
                    }
                    store8(a.out, a.g_fp32, idx, o);
                }
            }
        }
    }
    if (BWD) {
        if (active) {
            if (a.ddt_bias) {
#pragma unroll
                for (int e = 0; e < 8; ++e) atomicAdd(&a.ddt_bias[ch + e], dbias[e]);
            }
            if (a.dA_log) atomicAdd(&sDA[h - h_lo], dA);
        }
        __syncthreads();
        if (a.dA_log) {
            for (int i = threadIdx.x; i < 66; i += GATE_THREADS)
                if (h_lo + i < a.H && sDA[i] != 0.f) atomicAdd(&a.dA_log[h_lo + i], sDA[i]);
        }
    }
}

template <bool BWD>
__global__ void __launch_bounds__(GATE_THREADS) kda_beta_sigmoid_kernel(const void* x, int x_fp32, const float* dy, void* out,
                                                                       long long n) {
    for (long long i = (long long)blockIdx.x * GATE_THREADS + threadIdx.x; i < n; i += (long long)gridDim.x * GATE_THREADS) {
        const float xv = x_fp32 ? reinterpret_cast<const float*>(x)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
        const float y = __fdividef(1.f, 1.f + __expf(-xv));
        if (!BWD) {
            reinterpret_cast<float*>(out)[i] = y;
        } else {
            const float d = dy[i] * y * (1.f - y);
            if (x_fp32) reinterpret_cast<float*>(out)[i] = d;
            else reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(d);
        }
    }
}

}  // namespace kda

extern "C" int kda_launch_gate(const kda::GateArgs* a, int backward, cudaStream_t stream) {
    using namespace kda;
    if (a->M <= 0) return 0;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int groups = a->H * a->K / 8;
    const int gx = (groups + GATE_THREADS - 1) / GATE_THREADS;
    // about eight CTAs per SM in flight; the backward pass ends in one atomic per thread and channel, so it runs a
    // quarter as many, longer-lived CTAs
    long long gy = ((backward ? 2LL : 8LL) * sms + gx - 1) / gx;
    if (gy > a->M) gy = a->M;
    if (gy > 65535) gy = 65535;
    dim3 grid(gx, (unsigned)gy);
    if (backward) kda_gate_kernel<true><<<grid, GATE_THREADS, 0, stream>>>(*a);
    else kda_gate_kernel<false><<<grid, GATE_THREADS, 0, stream>>>(*a);
    return (int)cudaGetLastError();
}

extern "C" int kda_launch_beta_sigmoid(const void* x, int x_fp32, const float* dy, void* out, long long n, int backward,
                                       cudaStream_t stream) {
    using namespace kda;
    if (n <= 0) return 0;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long blocks = (n + GATE_THREADS - 1) / GATE_THREADS;
    if (blocks > 8LL * sms) blocks = 8LL * sms;
    if (backward) kda_beta_sigmoid_kernel<true><<<(unsigned)blocks, GATE_THREADS, 0, stream>>>(x, x_fp32, dy, out, n);
    else kda_beta_sigmoid_kernel<false><<<(unsigned)blocks, GATE_THREADS, 0, stream>>>(x, x_fp32, dy, out, n);
    return (int)cudaGetLastError();
}
