// Forward pass for callers that must not allocate device memory.
//
// cula_kda_fwd_intra / cula_kda_fwd_scan hand the per-(chunk, head) tile packs to each other through a buffer the
// caller allocates. Some callers cannot do that: a serving runtime that has already handed all of its device
// memory to its own pool, a plugin running inside someone else's memory-managed region, or code on a path where
// cudaMalloc's implicit device synchronisation is not acceptable. For them this file provides one extra entry
// point, cula_kda_fwd_noalloc, that keeps the tile packs in a fixed array living in the library's own device
// image. Inputs and outputs are still the caller's.
//
// Limits and rules
//   * at most CULA_KDA_NOALLOC_MAX_TILES (chunk, head) tiles per call, i.e. num_chunks * H <= 256
//     (for example 1024 tokens x 16 heads); larger problems are refused with CULA_KDA_ETOOBIG;
//   * the array (256 x 74,240 B = 18.1 MiB) is part of the module image: every GPU on which this library is
//     loaded holds it until the process exits;
//   * all calls on one device share the array and it keeps whatever the last call left in it. Nothing in it has
//     to start at zero (the first kernel writes every byte the second one reads), but two calls whose kernels
//     overlap on the GPU (different streams, or different host threads) race on it: serialise them;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress). Make that first
//     call before starting any stream capture on that device.
// The function calls no cudaMalloc / cudaFree and no allocating library routine.
#include <mutex>

#include "../../include/cula_kda.h"
#include "kda_common.cuh"
#include "kda_params.h"

extern "C" int kda_launch_fwd_intra(const kda::IntraParams* p, int num_chunks, cudaStream_t stream);
extern "C" int kda_launch_fwd_scan(const kda::ScanParams* p, cudaStream_t stream);

namespace {

constexpr int kMaxTiles = CULA_KDA_NOALLOC_MAX_TILES;
constexpr int kMaxDevices = 64;

// The scratch itself. In host code this name is only a handle for the runtime, NOT a device address:
// the address each GPU gave it is fetched once per device below and that pointer is what the kernels get.
static __device__ __align__(256) unsigned char g_tile_scratch[(size_t)kMaxTiles * kda::TP_BYTES];

std::mutex g_setup_mutex;
unsigned char* g_scratch_ptr[kMaxDevices] = {};

// Device address of g_tile_scratch on the current device (looked up on first use, then cached).
int scratch_for_current_device(unsigned char** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return CULA_KDA_EINVAL;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_tile_scratch);
        if (e != cudaSuccess) return (int)e;
        g_scratch_ptr[dev] = static_cast<unsigned char*>(ptr);
    }
    *out = g_scratch_ptr[dev];
    return 0;
}

inline bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

}  // namespace

extern "C" int cula_kda_noalloc_max_tiles(void) { return kMaxTiles; }

extern "C" int cula_kda_fwd_noalloc(const void* d_q, const void* d_k, const void* d_v, const void* d_g, int g_is_fp32,
                                    const void* d_beta, int beta_is_fp32, const float* d_A_log, const float* d_dt_bias,
                                    const float* d_h0, void* d_o, float* d_ht, const int* d_cu_seqlens,
                                    const int* d_chunk_indices, const int* d_chunk_offsets, int num_chunks, int N, int T,
                                    int H, float scale, int use_qk_l2norm, int gate_mode, float lower_bound,
                                    int* d_status, void* stream) {
    if (num_chunks == 0 || N == 0) return 0;
    if (!d_q || !d_k || !d_v || !d_g || !d_beta || !d_o || !d_status || num_chunks < 0 || N < 0 || H <= 0)
        return CULA_KDA_EINVAL;
    if (gate_mode < 0 || gate_mode > 2 || (gate_mode != 0 && !d_A_log)) return CULA_KDA_EINVAL;
    const bool varlen = d_cu_seqlens != nullptr;
    if (varlen != (d_chunk_indices != nullptr) || varlen != (d_chunk_offsets != nullptr)) return CULA_KDA_EINVAL;
    if (!varlen && (T <= 0 || num_chunks != N * ((T + kda::BT - 1) / kda::BT))) return CULA_KDA_EINVAL;
    if ((long long)num_chunks * H > kMaxTiles) return CULA_KDA_ETOOBIG;
    if (misaligned(d_q) || misaligned(d_k) || misaligned(d_v) || misaligned(d_g) || misaligned(d_o)) return CULA_KDA_EALIGN;

    unsigned char* tiles = nullptr;
    int rc = scratch_for_current_device(&tiles);
    if (rc != 0) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    kda::IntraParams ip{};
    ip.q = d_q; ip.k = d_k; ip.v = d_v; ip.g = d_g; ip.beta = d_beta; ip.A_log = d_A_log; ip.dt_bias = d_dt_bias;
    ip.cu_seqlens = d_cu_seqlens; ip.chunk_indices = d_chunk_indices; ip.tiles = tiles; ip.akk_out = nullptr;
    ip.mkk_out = nullptr; ip.status = d_status; ip.T = T; ip.H = H; ip.g_fp32 = g_is_fp32 & 1; ip.g_per_head = (g_is_fp32 >> 1) & 1; ip.beta_fp32 = beta_is_fp32 & 1; ip.beta_logit = (beta_is_fp32 >> 1) & 1;
    ip.use_l2norm = use_qk_l2norm; ip.gate_mode = gate_mode; ip.lower_bound = lower_bound; ip.scale = scale;
    rc = kda_launch_fwd_intra(&ip, num_chunks, s);
    if (rc != 0) return rc;

    kda::ScanParams sp{};
    sp.tiles = tiles; sp.h0 = d_h0; sp.o = d_o; sp.ht = d_ht; sp.h_out = nullptr; sp.vnew_out = nullptr; sp.h32_out = nullptr;
    sp.cu_seqlens = d_cu_seqlens; sp.chunk_offsets = d_chunk_offsets; sp.seq_order = nullptr; sp.status = d_status;
    sp.T = T; sp.H = H; sp.N = N;
    return kda_launch_fwd_scan(&sp, s);
}
