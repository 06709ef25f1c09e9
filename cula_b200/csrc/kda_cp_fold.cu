// Context parallelism: fold a chain of affine transitions into a state,
//     S <- h0 (or 0);   for j = 0 .. n-1:   S <- M_j S + C_j          (S, C_j: [128 x 128] per head; M_j: [128 x 128])
// Element j of the chain sits at c_all + j * stride and m_all + j * stride (floats), each [H, 128, 128] fp32, in THIS
// GPU's memory (the gathered buffers or the rank's own transitions); c_all == nullptr stands for C_j = 0, which
// turns the fold into the product of the M_j (used to compose the transitions of a shard's segments).
//
// One CTA per (head, 32-column slice of the state), fp32 CUDA-core arithmetic: M_j is brought into shared memory
// with cp.async one step ahead (double buffered), every thread owns 4 rows x 4 columns of the slice, and the inner loop
// issues 8 shared-memory loads per 64 FMAs. Counterpart of flash-linear-attention's merge kernel
// (fla/ops/cp/chunk_delta_h.py:321-457) reached from cula/kda/chunk_fwd.py:99-109.
#include "kda_common.cuh"

namespace kda {

constexpr int FOLD_COLS = 32;
constexpr int FOLD_THREADS = 256;
constexpr int FOLD_MS = 132;                                  // padded row of M in shared memory (floats)
constexpr int FOLD_SS = 36;                                   // padded row of the state slice
constexpr int FOLD_SMEM = (2 * DK * FOLD_MS + 2 * DK * FOLD_SS) * 4;

__device__ __forceinline__ void fold_cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}

__global__ void __launch_bounds__(FOLD_THREADS, 1) kda_cp_fold_kernel(const float* __restrict__ c_all, const float* __restrict__ m_all,
                                                                     const float* __restrict__ h0, float* __restrict__ s_out,
                                                                     int n, int H, size_t stride) {
    extern __shared__ __align__(16) float fsm[];
    float* sM = fsm;                                          // [2][128][FOLD_MS]
    float* sS = fsm + 2 * DK * FOLD_MS;                       // [2][128][FOLD_SS]
    const int h = blockIdx.x, v0 = blockIdx.y * FOLD_COLS;
    const int tid = threadIdx.x, kq = tid >> 3, c0 = 4 * (tid & 7);     // rows kq, kq+32, kq+64, kq+96; columns c0..c0+3
    const size_t head_off = (size_t)h * DK * DV;

    auto load_m = [&](int j, int buf) {
        const float* M = m_all + (size_t)j * stride + (size_t)h * DK * DK;
        for (int i = tid; i < DK * (DK / 4); i += FOLD_THREADS) {
            const int r = i >> 5, c4 = (i & 31) * 4;
            fold_cp_async16(sM + (size_t)buf * DK * FOLD_MS + r * FOLD_MS + c4, M + (size_t)r * DK + c4);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (n > 0) load_m(0, 0);
    for (int i = tid; i < DK * (FOLD_COLS / 4); i += FOLD_THREADS) {
        const int r = i >> 3, c4 = (i & 7) * 4;
        const float4 v = h0 ? *reinterpret_cast<const float4*>(h0 + head_off + (size_t)r * DV + v0 + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(sS + r * FOLD_SS + c4) = v;
    }
    int cur = 0;
    for (int j = 0; j < n; ++j) {
        if (j + 1 < n) {
            load_m(j + 1, (j + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                                      // M_j and the current state are visible to every thread
        const float* Mj = sM + (size_t)(j & 1) * DK * FOLD_MS;
        const float* Sc = sS + (size_t)cur * DK * FOLD_SS;
        float acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            float4 c = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c_all) c = *reinterpret_cast<const float4*>(c_all + (size_t)j * stride + head_off + (size_t)(kq + 32 * a) * DV + v0 + c0);
            acc[a][0] = c.x; acc[a][1] = c.y; acc[a][2] = c.z; acc[a][3] = c.w;
        }
#pragma unroll 2
        for (int mm = 0; mm < DK; mm += 4) {
            float mv[4][4], sv[4][4];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float4 t = *reinterpret_cast<const float4*>(Mj + (kq + 32 * a) * FOLD_MS + mm);
                mv[a][0] = t.x; mv[a][1] = t.y; mv[a][2] = t.z; mv[a][3] = t.w;
                const float4 u = *reinterpret_cast<const float4*>(Sc + (mm + a) * FOLD_SS + c0);
                sv[a][0] = u.x; sv[a][1] = u.y; sv[a][2] = u.z; sv[a][3] = u.w;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[a][e] = fmaf(mv[a][q], sv[q][e], acc[a][e]);
        }
        float* Sn = sS + (size_t)(cur ^ 1) * DK * FOLD_SS;
#pragma unroll
        for (int a = 0; a < 4; ++a)
            *reinterpret_cast<float4*>(Sn + (kq + 32 * a) * FOLD_SS + c0) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
        cur ^= 1;
        __syncthreads();                                      // the buffer of M_j may be overwritten by step j + 2
    }
    __syncthreads();
    for (int i = tid; i < DK * (FOLD_COLS / 4); i += FOLD_THREADS) {
        const int r = i >> 3, c4 = (i & 7) * 4;
        *reinterpret_cast<float4*>(s_out + head_off + (size_t)r * DV + v0 + c4) =
            *reinterpret_cast<const float4*>(sS + (size_t)cur * DK * FOLD_SS + r * FOLD_SS + c4);
    }
}

}  // namespace kda

extern "C" int kda_launch_cp_fold(const float* c_all, const float* m_all, const float* h0, float* s_out, int n, int H,
                                  long long stride_floats, cudaStream_t stream) {
    using namespace kda;
    cudaError_t e = cudaFuncSetAttribute(kda_cp_fold_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FOLD_SMEM);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(H, DV / FOLD_COLS);
    kda_cp_fold_kernel<<<grid, FOLD_THREADS, FOLD_SMEM, stream>>>(c_all, m_all, h0, s_out, n, H, (size_t)stride_floats);
    return (int)cudaGetLastError();
}
