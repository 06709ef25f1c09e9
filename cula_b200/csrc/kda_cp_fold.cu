// Context parallelism: fold the affine transitions of the predecessor shards into this rank's incoming state,
//     S <- h0 (or 0);   for j = 0 .. n_prev-1:   S <- M_j S + C_j
// with the gathered C_all [W, H, 128, 128] and M_all [W, H, 128, 128] (fp32) already in THIS GPU's memory.
// One CTA per (head, 32-column slice of the state); fp32 CUDA-core arithmetic (n_prev small products of 128^3 per
// head). Counterpart of flash-linear-attention's merge kernel (fla/ops/cp/chunk_delta_h.py:321-457) reached from
// cula/kda/chunk_fwd.py:99-109.
#include "kda_common.cuh"

namespace kda {

constexpr int FOLD_COLS = 32;

__global__ void __launch_bounds__(256) kda_cp_fold_kernel(const float* __restrict__ c_all, const float* __restrict__ m_all,
                                                          const float* __restrict__ h0, float* __restrict__ s_in,
                                                          int n_prev, int H) {
    __shared__ float sS[2][DK][FOLD_COLS + 1];
    const int h = blockIdx.x, v0 = blockIdx.y * FOLD_COLS;
    const int tid = threadIdx.x, k = tid >> 1, c0 = (tid & 1) * 16;
    const size_t head_off = (size_t)h * DK * DV;
    for (int i = tid; i < DK * FOLD_COLS; i += 256) {
        const int r = i / FOLD_COLS, c = i % FOLD_COLS;
        sS[0][r][c] = h0 ? h0[head_off + (size_t)r * DV + v0 + c] : 0.f;
    }
    __syncthreads();
    int cur = 0;
    for (int j = 0; j < n_prev; ++j) {
        const float* M = m_all + ((size_t)j * H + h) * DK * DK + (size_t)k * DK;
        const float* C = c_all + ((size_t)j * H + h) * DK * DV + (size_t)k * DV + v0 + c0;
        float acc[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[e] = C[e];
        for (int mm = 0; mm < DK; mm += 4) {
            const float4 mv = *reinterpret_cast<const float4*>(M + mm);
            const float mvv[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int e = 0; e < 16; ++e) acc[e] = fmaf(mvv[q], sS[cur][mm + q][c0 + e], acc[e]);
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) sS[cur ^ 1][k][c0 + e] = acc[e];
        __syncthreads();
        cur ^= 1;
    }
    for (int i = tid; i < DK * FOLD_COLS; i += 256) {
        const int r = i / FOLD_COLS, c = i % FOLD_COLS;
        s_in[head_off + (size_t)r * DV + v0 + c] = sS[cur][r][c];
    }
}

}  // namespace kda

extern "C" int kda_launch_cp_fold(const float* c_all, const float* m_all, const float* h0, float* s_in, int n_prev, int H,
                                  cudaStream_t stream) {
    dim3 grid(H, kda::DV / kda::FOLD_COLS);
    kda::kda_cp_fold_kernel<<<grid, 256, 0, stream>>>(c_all, m_all, h0, s_in, n_prev, H);
    return (int)cudaGetLastError();
}
