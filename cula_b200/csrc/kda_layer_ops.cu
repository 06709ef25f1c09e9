// The two layer operators on either side of chunk_kda in a Kimi-Linear block, as stand-alone streaming kernels:
//   short causal depthwise convolution + SiLU on the q / k / v projections (kernel width <= 4), forward and backward,
//   gated RMS norm on the attention output, y = rmsnorm(x) * w * act(g), forward and backward.
// They replace flash-linear-attention's ShortConvolution / causal_conv1d (fla/modules/convolution.py) and
// FusedRMSNormGated / rms_norm_gated (fla/modules/fused_norm_gate.py:35-120, 846-869), which the layer that calls the
// reference's chunk_kda uses (fla/layers/kda.py:147-165, 191, 306). HBM-bound: each element is read and written once
// (the convolution re-reads a 3-token halo per 64-token chunk).
#include "kda_common.cuh"
#include "kda_params.h"

namespace kda {

constexpr int LO_THREADS = 128;
constexpr int CONV_MAXW = 4;

__device__ __forceinline__ void lo_load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    float2 f;
    f = unpack_bf16(a.x); v[0] = f.x; v[1] = f.y;
    f = unpack_bf16(a.y); v[2] = f.x; v[3] = f.y;
    f = unpack_bf16(a.z); v[4] = f.x; v[5] = f.y;
    f = unpack_bf16(a.w); v[6] = f.x; v[7] = f.y;
}
__device__ __forceinline__ void lo_unpack8(const uint4& a, float (&v)[8]) {
    float2 f;
    f = unpack_bf16(a.x); v[0] = f.x; v[1] = f.y;
    f = unpack_bf16(a.y); v[2] = f.x; v[3] = f.y;
    f = unpack_bf16(a.z); v[4] = f.x; v[5] = f.y;
    f = unpack_bf16(a.w); v[6] = f.x; v[7] = f.y;
}
__device__ __forceinline__ void lo_store8(__nv_bfloat16* p, const float (&v)[8]) {
    *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// ------------------------------------------------------------------------------------------------------------------
// Causal depthwise convolution: pre[t, d] = bias[d] + sum_i w[d, i] x[t - (W-1) + i, d],  y = silu(pre) (or pre).
// Tokens before the start of a sequence come from cache[n, d, :] (the last W inputs of the previous call, newest
// last) or are zero. One CTA column per 64-token chunk (chunks never straddle sequences: the same tables as the
// attention kernels), one thread per 8 channels; the thread walks its chunk with a sliding window in registers.
// ------------------------------------------------------------------------------------------------------------------

__device__ __forceinline__ void conv_load_row(const ConvArgs& a, int seq, int seq_start, int t, int ch, float (&v)[8]) {
    // token t of the flattened axis, or (t < seq_start) the cached inputs of the previous call, or zero
    if (t >= seq_start) {
        lo_load8(a.x + (size_t)t * a.D + ch, v);
    } else if (a.cache_in && seq_start - t <= a.W) {
        const float* c = a.cache_in + ((size_t)seq * a.D + ch) * a.W + (a.W - (seq_start - t));
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = c[e * a.W];
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = 0.f;
    }
}

template <bool BWD>
__global__ void __launch_bounds__(LO_THREADS) kda_short_conv_kernel(const ConvArgs a) {
    const int ch = 8 * (blockIdx.x * LO_THREADS + threadIdx.x);
    if (ch >= a.D) return;
    const ChunkInfo ci = chunk_info(blockIdx.y, a.cu_seqlens, a.chunk_indices, a.T);
    const int seq_start = a.cu_seqlens ? a.cu_seqlens[ci.seq] : ci.seq * a.T;
    const int seq_end = a.cu_seqlens ? a.cu_seqlens[ci.seq + 1] : (ci.seq + 1) * a.T;
    const int W = a.W, t0 = ci.row0, t1 = ci.row0 + ci.valid;
    // w: the taps, zero beyond W. wr: the same taps right-aligned in a window of CONV_MAXW slots (wr[e][k] multiplies
    // window slot k), so that every index into the register arrays below is a compile-time constant whatever W is --
    // an index that depends on W would put the window into local memory
    float w[8][CONV_MAXW], wr[8][CONV_MAXW], b[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        if (W == CONV_MAXW) {      // the usual width: one 16-byte load per channel, both alignments coincide
            const float4 v = *reinterpret_cast<const float4*>(a.w + (size_t)(ch + e) * CONV_MAXW);
            w[e][0] = wr[e][0] = v.x; w[e][1] = wr[e][1] = v.y; w[e][2] = wr[e][2] = v.z; w[e][3] = wr[e][3] = v.w;
        } else {
#pragma unroll
            for (int i = 0; i < CONV_MAXW; ++i) {
                w[e][i] = i < W ? a.w[(size_t)(ch + e) * W + i] : 0.f;
                const int tap = i - (CONV_MAXW - W);
                wr[e][i] = tap >= 0 ? a.w[(size_t)(ch + e) * W + tap] : 0.f;
            }
        }
        b[e] = a.bias ? a.bias[ch + e] : 0.f;
    }
    // window[k] = x[t - (CONV_MAXW-1) + k]; tap i of a width-W kernel multiplies window[CONV_MAXW - W + i]
    float win[CONV_MAXW][8];
#pragma unroll
    for (int k = 0; k < CONV_MAXW - 1; ++k) conv_load_row(a, ci.seq, seq_start, t0 - (CONV_MAXW - 1) + k, ch, win[k + 1]);
    if (!BWD) {
        // the rows of eight tokens are requested before the first of them is used (a thread walks its chunk serially:
        // one load per step would pay a full memory latency per token); rows past the chunk re-read its last row
        constexpr int NB = 8;
        for (int tb = t0; tb < t1; tb += NB) {
            uint4 raw[NB];
#pragma unroll
            for (int i = 0; i < NB; ++i)
                raw[i] = *reinterpret_cast<const uint4*>(a.x + (size_t)min(tb + i, t1 - 1) * a.D + ch);
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const int t = tb + i;
                if (t < t1) {
#pragma unroll
                    for (int k = 0; k < CONV_MAXW - 1; ++k)
#pragma unroll
                        for (int e = 0; e < 8; ++e) win[k][e] = win[k + 1][e];
                    lo_unpack8(raw[i], win[CONV_MAXW - 1]);
                    float o[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        float pre = b[e];
#pragma unroll
                        for (int k = 0; k < CONV_MAXW; ++k) pre = fmaf(wr[e][k], win[k][e], pre);
                        o[e] = a.silu ? pre * sigmoid_f(pre) : pre;
                    }
                    lo_store8(a.y + (size_t)t * a.D + ch, o);
                }
            }
        }
        if (a.cache_out && t1 == seq_end) {      // the last W inputs of the sequence, newest last, zero-padded on the left
            float* c = a.cache_out + ((size_t)ci.seq * a.D + ch) * W;
#pragma unroll
            for (int k = 0; k < CONV_MAXW; ++k) {
                const int tap = k - (CONV_MAXW - W);
                if (tap >= 0) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) c[e * W + tap] = win[k][e];
                }
            }
        }
    } else {
        // walk three tokens past the chunk (inside the sequence): dx[u] = sum_i w[i] dpre[u + (W-1) - i] needs them
        float dwin[CONV_MAXW][8];       // dwin[k] = dpre[t - (CONV_MAXW-1) + k]
        float dw_acc[8][CONV_MAXW], db_acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            db_acc[e] = 0.f;
#pragma unroll
            for (int i = 0; i < CONV_MAXW; ++i) dw_acc[e][i] = dwin[i][e] = 0.f;
        }
        constexpr int NBB = 4;          // rows of four tokens (x and dy) in flight before the first is used
        const int t_end = t1 + (W - 1), t_last = seq_end - 1;
        for (int tb = t0; tb < t_end; tb += NBB) {
          uint4 raw_x[NBB], raw_dy[NBB];
#pragma unroll
          for (int i = 0; i < NBB; ++i) {
              const size_t off = (size_t)min(tb + i, t_last) * a.D + ch;      // clamped: tokens past the sequence are not used
              raw_x[i] = *reinterpret_cast<const uint4*>(a.x + off);
              raw_dy[i] = *reinterpret_cast<const uint4*>(a.dy + off);
          }
#pragma unroll
          for (int i = 0; i < NBB; ++i) {
            const int t = tb + i;
            if (t >= t_end) break;
#pragma unroll
            for (int k = 0; k < CONV_MAXW - 1; ++k)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    win[k][e] = win[k + 1][e];
                    dwin[k][e] = dwin[k + 1][e];
                }
            const bool live = t < seq_end;
            float dyv[8];
            if (live) {
                lo_unpack8(raw_x[i], win[CONV_MAXW - 1]);
                lo_unpack8(raw_dy[i], dyv);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float dp = 0.f;
                if (live) {
                    float pre = b[e];
#pragma unroll
                    for (int k = 0; k < CONV_MAXW; ++k) pre = fmaf(wr[e][k], win[k][e], pre);
                    const float s = sigmoid_f(pre);
                    dp = a.silu ? dyv[e] * s * (1.f + pre * (1.f - s)) : dyv[e];
                    if (t < t1) {            // parameter gradients: each token counted once, by its own chunk
                        db_acc[e] += dp;
#pragma unroll
                        for (int k = 0; k < CONV_MAXW; ++k) dw_acc[e][k] = fmaf(dp, win[k][e], dw_acc[e][k]);     // by window slot
                    }
                }
                dwin[CONV_MAXW - 1][e] = dp;
            }
            const int u = t - (W - 1);
            if (u >= t0 && u < t1) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float acc = 0.f;
#pragma unroll
                    for (int i = 0; i < CONV_MAXW; ++i)
                        if (i < W) acc = fmaf(w[e][i], dwin[CONV_MAXW - 1 - i][e], acc);     // dpre[u + (W-1) - i] = dpre[t - i]
                    o[e] = acc;
                }
                lo_store8(a.dx + (size_t)u * a.D + ch, o);
            }
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
#pragma unroll
            for (int k = 0; k < CONV_MAXW; ++k) {
                const int tap = k - (CONV_MAXW - W);
                if (tap >= 0) atomicAdd(&a.dw[(size_t)(ch + e) * W + tap], dw_acc[e][k]);
            }
            if (a.dbias) atomicAdd(&a.dbias[ch + e], db_acc[e]);
        }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// Gated RMS norm over rows of D elements (D a multiple of 256, <= 1024... or 128): one warp per row.
//   n = x * rstd, rstd = rsqrt(mean(x^2) + eps);  y = n * w * act(g), act = sigmoid or swish.
// ------------------------------------------------------------------------------------------------------------------

template <int VPL, bool BWD>       // VPL: 8-element vectors per lane (D = 256 * VPL), or D = 128 with half of ... see launcher
__global__ void __launch_bounds__(LO_THREADS) kda_rms_norm_gated_kernel(const NormArgs a) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (long long)blockIdx.x * (LO_THREADS / 32) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (LO_THREADS / 32);
    const int per_lane = a.D / 32;                 // 4 (D = 128) or 8 * VPL
    const bool narrow = per_lane == 4;
    float wv[VPL][8], dw_acc[VPL][8];
#pragma unroll
    for (int v = 0; v < VPL; ++v)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int col = narrow ? 4 * lane + (e & 3) : 256 * v + 8 * lane + e;
            wv[v][e] = a.w[col];
            dw_acc[v][e] = 0.f;
        }
    // Rows are taken NB at a time per warp and all their loads are issued before the first is used (a warp has dozens
    // of rows and one row per dependent step would pay a full memory latency each).
    constexpr int NB = VPL == 1 ? 4 : (VPL == 2 ? 2 : 1);
    for (long long rb = warp0; rb < a.R; rb += (long long)NB * nwarps) {
      uint4 rx[NB][VPL], rg[NB][VPL], rd[NB][VPL];
#pragma unroll
      for (int i = 0; i < NB; ++i) {
        const size_t base = (size_t)min(rb + (long long)i * nwarps, a.R - 1) * a.D;       // clamped: surplus rows are not used
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            if (narrow) {
                const uint2 x2 = *reinterpret_cast<const uint2*>(a.x + base + 4 * lane);
                const uint2 g2 = *reinterpret_cast<const uint2*>(a.g + base + 4 * lane);
                rx[i][v] = make_uint4(x2.x, x2.y, 0u, 0u);
                rg[i][v] = make_uint4(g2.x, g2.y, 0u, 0u);
                if (BWD) {
                    const uint2 d2 = *reinterpret_cast<const uint2*>(a.dy + base + 4 * lane);
                    rd[i][v] = make_uint4(d2.x, d2.y, 0u, 0u);
                }
            } else {
                rx[i][v] = *reinterpret_cast<const uint4*>(a.x + base + 256 * v + 8 * lane);
                rg[i][v] = *reinterpret_cast<const uint4*>(a.g + base + 256 * v + 8 * lane);
                if (BWD) rd[i][v] = *reinterpret_cast<const uint4*>(a.dy + base + 256 * v + 8 * lane);
            }
        }
      }
#pragma unroll
      for (int i = 0; i < NB; ++i) {
        const long long row = rb + (long long)i * nwarps;
        if (row >= a.R) break;
        const size_t base = (size_t)row * a.D;
        float xv[VPL][8], gv[VPL][8];
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            lo_unpack8(rx[i][v], xv[v]);      // narrow rows: the upper half of the 8-wide vectors is zero
            lo_unpack8(rg[i][v], gv[v]);
        }
        float rstd;
        if (!BWD) {
            float ss = 0.f;
#pragma unroll
            for (int v = 0; v < VPL; ++v)
#pragma unroll
                for (int e = 0; e < 8; ++e) ss = fmaf(xv[v][e], xv[v][e], ss);
#pragma unroll
            for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            rstd = rsqrtf(ss / (float)a.D + a.eps);
            if (lane == 0) a.rstd[row] = rstd;
        } else {
            rstd = a.rstd[row];
        }
        float out[VPL][8];
        if (!BWD) {
#pragma unroll
            for (int v = 0; v < VPL; ++v)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float s = sigmoid_f(gv[v][e]);
                    out[v][e] = xv[v][e] * rstd * wv[v][e] * (a.swish ? gv[v][e] * s : s);
                }
        } else {
            float dyv[VPL][8], dn[VPL][8], dgo[VPL][8], dot = 0.f;
#pragma unroll
            for (int v = 0; v < VPL; ++v) lo_unpack8(rd[i][v], dyv[v]);
#pragma unroll
            for (int v = 0; v < VPL; ++v)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float gg = gv[v][e], s = sigmoid_f(gg), n = xv[v][e] * rstd;
                    const float act = a.swish ? gg * s : s;
                    const float dact = a.swish ? s * (1.f + gg * (1.f - s)) : s * (1.f - s);
                    const float z = n * wv[v][e];
                    const float dz = dyv[v][e] * act;
                    dgo[v][e] = dyv[v][e] * z * dact;
                    dw_acc[v][e] = fmaf(dz, n, dw_acc[v][e]);
                    dn[v][e] = dz * wv[v][e];
                    dot = fmaf(dn[v][e], n, dot);
                }
#pragma unroll
            for (int o = 16; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            const float mean_dot = dot / (float)a.D;
#pragma unroll
            for (int v = 0; v < VPL; ++v)
#pragma unroll
                for (int e = 0; e < 8; ++e) out[v][e] = rstd * (dn[v][e] - xv[v][e] * rstd * mean_dot);
            if (narrow) {
                *reinterpret_cast<uint2*>(a.dg + base + 4 * lane) = make_uint2(pack_bf16(dgo[0][0], dgo[0][1]), pack_bf16(dgo[0][2], dgo[0][3]));
            } else {
#pragma unroll
                for (int v = 0; v < VPL; ++v) lo_store8(a.dg + base + 256 * v + 8 * lane, dgo[v]);
            }
        }
        __nv_bfloat16* dst = BWD ? a.dx : a.y;
        if (narrow) {
            *reinterpret_cast<uint2*>(dst + base + 4 * lane) = make_uint2(pack_bf16(out[0][0], out[0][1]), pack_bf16(out[0][2], out[0][3]));
        } else {
#pragma unroll
            for (int v = 0; v < VPL; ++v) lo_store8(dst + base + 256 * v + 8 * lane, out[v]);
        }
      }
    }
    if (BWD) {
        // the weight gradient: the CTA's warps are summed in shared memory first, then one global atomic per column and CTA
        __shared__ float s_dw[1024];
        for (int c = threadIdx.x; c < a.D; c += LO_THREADS) s_dw[c] = 0.f;
        __syncthreads();
#pragma unroll
        for (int v = 0; v < VPL; ++v)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                if (narrow && e >= 4) continue;
                const int col = narrow ? 4 * lane + e : 256 * v + 8 * lane + e;
                atomicAdd(&s_dw[col], dw_acc[v][e]);
            }
        __syncthreads();
        for (int c = threadIdx.x; c < a.D; c += LO_THREADS) atomicAdd(&a.dw[c], s_dw[c]);
    }
}

}  // namespace kda

extern "C" int kda_launch_short_conv(const kda::ConvArgs* a, int num_chunks, int backward, cudaStream_t stream) {
    using namespace kda;
    if (num_chunks <= 0) return 0;
    dim3 grid((a->D / 8 + LO_THREADS - 1) / LO_THREADS, num_chunks);
    if (backward) kda_short_conv_kernel<true><<<grid, LO_THREADS, 0, stream>>>(*a);
    else kda_short_conv_kernel<false><<<grid, LO_THREADS, 0, stream>>>(*a);
    return (int)cudaGetLastError();
}

extern "C" int kda_launch_rms_norm_gated(const kda::NormArgs* a, int backward, cudaStream_t stream) {
    using namespace kda;
    if (a->R <= 0) return 0;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long blocks = (a->R + LO_THREADS / 32 - 1) / (LO_THREADS / 32);
    const long long cap = (backward ? 4LL : 16LL) * sms;     // backward: fewer, longer-lived CTAs keep the dw atomics few
    if (blocks > cap) blocks = cap;
    const int vpl = a->D == 128 ? 1 : a->D / 256;
#define KDA_NORM_LAUNCH(V)                                                                                        \
    do {                                                                                                          \
        if (backward) kda_rms_norm_gated_kernel<V, true><<<(unsigned)blocks, LO_THREADS, 0, stream>>>(*a);          \
        else kda_rms_norm_gated_kernel<V, false><<<(unsigned)blocks, LO_THREADS, 0, stream>>>(*a);                  \
    } while (0)
    if (vpl == 1) KDA_NORM_LAUNCH(1);
    else if (vpl == 2) KDA_NORM_LAUNCH(2);
    else if (vpl == 4) KDA_NORM_LAUNCH(4);
    else return -1;
#undef KDA_NORM_LAUNCH
    return (int)cudaGetLastError();
}
