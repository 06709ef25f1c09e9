// C-ABI layer: argument checks, parameter structs, launches. No torch types, no allocation.
#include "../../include/cula_kda.h"
#include "kda_common.cuh"
#include "kda_params.h"

extern "C" int kda_launch_fwd_intra(const kda::IntraParams* p, int num_chunks, cudaStream_t stream);
extern "C" int kda_launch_fwd_scan(const kda::ScanParams* p, cudaStream_t stream);

namespace {
inline bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }
}

extern "C" int kda_fwd_intra_smem_bytes();
extern "C" int kda_fwd_scan_smem_bytes();

extern "C" int cula_kda_tile_pack_bytes(void) { return kda::TP_BYTES; }
extern "C" int cula_kda_fwd_intra_smem_bytes(void) { return kda_fwd_intra_smem_bytes(); }
extern "C" int cula_kda_fwd_scan_smem_bytes(void) { return kda_fwd_scan_smem_bytes(); }

extern "C" int cula_kda_fwd_intra(const void* d_q, const void* d_k, const void* d_v, const void* d_g, int g_is_fp32,
                                  const void* d_beta, int beta_is_fp32, const float* d_A_log, const float* d_dt_bias,
                                  const int* d_cu_seqlens, const int* d_chunk_indices, int num_chunks, int T, int H,
                                  float scale, int use_qk_l2norm, int gate_mode, float lower_bound, void* d_tiles,
                                  float* d_akk, int* d_status, void* stream) {
    if (num_chunks == 0) return 0;
    if (!d_q || !d_k || !d_v || !d_g || !d_beta || !d_tiles || !d_status || num_chunks < 0 || H <= 0) return CULA_KDA_EINVAL;
    if (gate_mode < 0 || gate_mode > 2 || (gate_mode != 0 && !d_A_log)) return CULA_KDA_EINVAL;
    if ((d_cu_seqlens == nullptr) != (d_chunk_indices == nullptr)) return CULA_KDA_EINVAL;
    if (!d_cu_seqlens && T <= 0) return CULA_KDA_EINVAL;
    if (misaligned(d_q) || misaligned(d_k) || misaligned(d_v) || misaligned(d_g) || misaligned(d_tiles) ||
        misaligned(d_akk))
        return CULA_KDA_EALIGN;
    kda::IntraParams p{};
    p.q = d_q; p.k = d_k; p.v = d_v; p.g = d_g; p.beta = d_beta;
    p.A_log = d_A_log; p.dt_bias = d_dt_bias;
    p.cu_seqlens = d_cu_seqlens; p.chunk_indices = d_chunk_indices;
    p.tiles = static_cast<unsigned char*>(d_tiles);
    p.akk_out = d_akk;
    p.status = d_status;
    p.T = T; p.H = H; p.g_fp32 = g_is_fp32; p.beta_fp32 = beta_is_fp32;
    p.use_l2norm = use_qk_l2norm; p.gate_mode = gate_mode; p.lower_bound = lower_bound; p.scale = scale;
    return kda_launch_fwd_intra(&p, num_chunks, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_fwd_scan(const void* d_tiles, const float* d_h0, void* d_o, float* d_ht, void* d_h_out,
                                 void* d_vnew_out, const int* d_cu_seqlens, const int* d_chunk_offsets,
                                 const int* d_seq_order, int N, int T, int H, int* d_status, void* stream) {
    if (N == 0) return 0;
    if (!d_tiles || !d_o || !d_status || N < 0 || H <= 0) return CULA_KDA_EINVAL;
    if ((d_cu_seqlens == nullptr) != (d_chunk_offsets == nullptr)) return CULA_KDA_EINVAL;
    if (!d_cu_seqlens && T <= 0) return CULA_KDA_EINVAL;
    if ((d_h_out == nullptr) != (d_vnew_out == nullptr)) return CULA_KDA_EINVAL;
    if (misaligned(d_tiles) || misaligned(d_o) || misaligned(d_h_out) || misaligned(d_vnew_out)) return CULA_KDA_EALIGN;
    kda::ScanParams p{};
    p.tiles = static_cast<const unsigned char*>(d_tiles);
    p.h0 = d_h0; p.o = d_o; p.ht = d_ht; p.h_out = d_h_out; p.vnew_out = d_vnew_out;
    p.cu_seqlens = d_cu_seqlens; p.chunk_offsets = d_chunk_offsets; p.seq_order = d_seq_order;
    p.status = d_status; p.T = T; p.H = H; p.N = N;
    return kda_launch_fwd_scan(&p, static_cast<cudaStream_t>(stream));
}

extern "C" const char* cula_kda_strerror(int code) {
    if (code == 0) return "ok";
    if (code == CULA_KDA_EINVAL) return "invalid argument (null pointer, non-positive size or bad enum)";
    if (code == CULA_KDA_EALIGN) return "pointer is not 16-byte aligned";
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown error";
}
