// C-ABI layer: argument checks, parameter structs, launches. No torch types, no allocation.
#include "../../include/cula_kda.h"
#include "kda_common.cuh"
#include "kda_params.h"

extern "C" int kda_launch_fwd_intra(const kda::IntraParams* p, int num_chunks, cudaStream_t stream);
extern "C" int kda_launch_fwd_scan(const kda::ScanParams* p, cudaStream_t stream);
extern "C" int kda_launch_fwd_transition(const kda::ScanParams* p, cudaStream_t stream);
extern "C" int kda_launch_cp_fold(const float* c_all, const float* m_all, const float* h0, float* s_out, int n, int H,
                                  long long stride_floats, cudaStream_t stream);
extern "C" int kda_launch_grad_scale(const void* d_o, size_t n_do, const float* dht, size_t n_dht, unsigned int* amax_bits,
                                     float* gscale, cudaStream_t stream);
extern "C" int kda_launch_bwd_scan(const kda::BwdScanParams* p, cudaStream_t stream);
extern "C" int kda_launch_bwd_dense(const kda::BwdDenseParams* p, int num_chunks, cudaStream_t stream);
extern "C" int kda_launch_bwd_gated(const kda::BwdGatedParams* p, int num_chunks, cudaStream_t stream);

namespace {
inline bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }
}

extern "C" int kda_launch_decode(const void* q, const void* k, const void* v, const void* a, int a_fp32, const void* b, int b_fp32,
                                 const float* A_log, const float* dt_bias, float* state, const int* indices, void* o,
                                 int N, int H, int HV, int V, int pool, float scale, int use_l2norm, float softplus_beta,
                                 float softplus_threshold, int state_kv, int* status, cudaStream_t stream);
extern "C" int kda_fwd_intra_smem_bytes();
extern "C" int kda_fwd_scan_smem_bytes();

extern "C" int cula_kda_tile_pack_bytes(void) { return kda::TP_BYTES; }
extern "C" int cula_kda_fwd_intra_smem_bytes(void) { return kda_fwd_intra_smem_bytes(); }
extern "C" int cula_kda_fwd_scan_smem_bytes(void) { return kda_fwd_scan_smem_bytes(); }

extern "C" int cula_kda_fwd_intra(const void* d_q, const void* d_k, const void* d_v, const void* d_g, int g_is_fp32,
                                  const void* d_beta, int beta_is_fp32, const float* d_A_log, const float* d_dt_bias,
                                  const int* d_cu_seqlens, const int* d_chunk_indices, int num_chunks, int T, int H,
                                  float scale, int use_qk_l2norm, int gate_mode, float lower_bound, void* d_tiles,
                                  float* d_akk, float* d_mkk, int* d_status, void* stream) {
    if (num_chunks == 0) return 0;
    if (!d_q || !d_k || !d_v || !d_g || !d_beta || !d_tiles || !d_status || num_chunks < 0 || H <= 0) return CULA_KDA_EINVAL;
    if (gate_mode < 0 || gate_mode > 2 || (gate_mode != 0 && !d_A_log)) return CULA_KDA_EINVAL;
    if ((d_cu_seqlens == nullptr) != (d_chunk_indices == nullptr)) return CULA_KDA_EINVAL;
    if (!d_cu_seqlens && T <= 0) return CULA_KDA_EINVAL;
    if (misaligned(d_q) || misaligned(d_k) || misaligned(d_v) || misaligned(d_tiles) || misaligned(d_akk) || misaligned(d_mkk) ||
        (!(g_is_fp32 & CULA_KDA_G_PER_HEAD) && misaligned(d_g)))
        return CULA_KDA_EALIGN;
    if (g_is_fp32 & ~(CULA_KDA_G_FP32 | CULA_KDA_G_PER_HEAD)) return CULA_KDA_EINVAL;
    kda::IntraParams p{};
    p.q = d_q; p.k = d_k; p.v = d_v; p.g = d_g; p.beta = d_beta;
    p.A_log = d_A_log; p.dt_bias = d_dt_bias;
    p.cu_seqlens = d_cu_seqlens; p.chunk_indices = d_chunk_indices;
    p.tiles = static_cast<unsigned char*>(d_tiles);
    p.akk_out = d_akk;
    p.mkk_out = d_mkk;
    p.status = d_status;
    p.T = T; p.H = H; p.g_fp32 = g_is_fp32 & CULA_KDA_G_FP32; p.g_per_head = (g_is_fp32 & CULA_KDA_G_PER_HEAD) != 0;
    p.beta_fp32 = beta_is_fp32 & CULA_KDA_BETA_FP32; p.beta_logit = (beta_is_fp32 & CULA_KDA_BETA_LOGIT) != 0;
    p.use_l2norm = use_qk_l2norm; p.gate_mode = gate_mode; p.lower_bound = lower_bound; p.scale = scale;
    return kda_launch_fwd_intra(&p, num_chunks, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_fwd_scan(const void* d_tiles, const float* d_h0, void* d_o, float* d_ht, void* d_h_out,
                                 void* d_vnew_out, float* d_h32_out, const int* d_cu_seqlens, const int* d_chunk_offsets,
                                 const int* d_seq_order, int N, int T, int H, int* d_status, void* stream) {
    if (N == 0) return 0;
    if (!d_tiles || !d_status || N < 0 || H <= 0) return CULA_KDA_EINVAL;
    if (!d_o && !d_vnew_out) return CULA_KDA_EINVAL;      // nothing to produce
    if ((d_cu_seqlens == nullptr) != (d_chunk_offsets == nullptr)) return CULA_KDA_EINVAL;
    if (!d_cu_seqlens && T <= 0) return CULA_KDA_EINVAL;
    if ((d_h_out || d_h32_out) && !d_vnew_out) return CULA_KDA_EINVAL;
    if (misaligned(d_tiles) || misaligned(d_o) || misaligned(d_h_out) || misaligned(d_vnew_out)) return CULA_KDA_EALIGN;
    kda::ScanParams p{};
    p.tiles = static_cast<const unsigned char*>(d_tiles);
    p.h0 = d_h0; p.o = d_o; p.ht = d_ht; p.h_out = d_h_out; p.vnew_out = d_vnew_out; p.h32_out = d_h32_out;
    p.cu_seqlens = d_cu_seqlens; p.chunk_offsets = d_chunk_offsets; p.seq_order = d_seq_order;
    p.status = d_status; p.T = T; p.H = H; p.N = N;
    return kda_launch_fwd_scan(&p, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_cp_transition(const void* d_tiles, float* d_c_out, float* d_m_out, const int* d_cu_seqlens,
                                      const int* d_chunk_offsets, int N, int T, int H, int* d_status, void* stream) {
    if (N == 0) return 0;
    if (!d_tiles || !d_c_out || !d_m_out || !d_status || N < 0 || H <= 0) return CULA_KDA_EINVAL;
    if ((d_cu_seqlens == nullptr) != (d_chunk_offsets == nullptr)) return CULA_KDA_EINVAL;
    if (!d_cu_seqlens && T <= 0) return CULA_KDA_EINVAL;
    if (misaligned(d_tiles)) return CULA_KDA_EALIGN;
    kda::ScanParams p{};
    p.tiles = static_cast<const unsigned char*>(d_tiles);
    p.ht = d_c_out; p.m_out = d_m_out; p.cu_seqlens = d_cu_seqlens; p.chunk_offsets = d_chunk_offsets;
    p.status = d_status; p.T = T; p.H = H; p.N = N;
    return kda_launch_fwd_transition(&p, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_cp_fold(const float* d_c_all, const float* d_m_all, const float* d_h0, float* d_s_out, int n,
                                int H, long long stride_floats, void* stream) {
    if (!d_s_out || n < 0 || H <= 0 || (n > 0 && !d_m_all)) return CULA_KDA_EINVAL;
    if (stride_floats <= 0) stride_floats = (long long)H * kda::DK * kda::DV;
    if (misaligned(d_m_all) || misaligned(d_c_all) || misaligned(d_h0) || misaligned(d_s_out) || (stride_floats & 3))
        return CULA_KDA_EALIGN;
    return kda_launch_cp_fold(d_c_all, d_m_all, d_h0, d_s_out, n, H, stride_floats, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_decode(const void* d_q, const void* d_k, const void* d_v, const void* d_a, int a_is_fp32,
                               const void* d_b, int b_is_fp32, const float* d_A_log, const float* d_dt_bias,
                               float* d_state, const int* d_state_indices, void* d_o, int N, int H, int HV, int V,
                               int pool_size, float scale, int use_qk_l2norm, float softplus_beta,
                               float softplus_threshold, int state_is_kv, int* d_status, void* stream) {
    if (N == 0) return 0;
    if (!d_q || !d_k || !d_v || !d_a || !d_b || !d_A_log || !d_state || !d_o || !d_status) return CULA_KDA_EINVAL;
    if (N < 0 || H <= 0 || HV <= 0 || HV % H != 0 || V <= 0 || V % 32 != 0 || pool_size <= 0) return CULA_KDA_EINVAL;
    if (!(softplus_beta > 0.f)) return CULA_KDA_EINVAL;
    if (!d_state_indices && pool_size < N) return CULA_KDA_EINVAL;
    if (misaligned(d_q) || misaligned(d_k) || misaligned(d_state)) return CULA_KDA_EALIGN;
    return kda_launch_decode(d_q, d_k, d_v, d_a, a_is_fp32, d_b, b_is_fp32, d_A_log, d_dt_bias, d_state, d_state_indices, d_o,
                             N, H, HV, V, pool_size, scale, use_qk_l2norm, softplus_beta, softplus_threshold, state_is_kv,
                             d_status, static_cast<cudaStream_t>(stream));
}

// ---- host-side index tables for a packed batch (plain host memory in, plain host memory out) ----
extern "C" int cula_kda_num_chunks(const int* h_cu_seqlens, int N) {
    if (!h_cu_seqlens || N < 0 || h_cu_seqlens[0] != 0) return CULA_KDA_EINVAL;
    long long total = 0;
    for (int n = 0; n < N; ++n) {
        const int len = h_cu_seqlens[n + 1] - h_cu_seqlens[n];
        if (len < 0) return CULA_KDA_EINVAL;
        total += (len + kda::BT - 1) / kda::BT;
    }
    return total > 0x7fffffffLL ? CULA_KDA_ETOOBIG : (int)total;
}

extern "C" int cula_kda_build_chunk_tables(const int* h_cu_seqlens, int N, int* h_chunk_indices, int* h_chunk_offsets,
                                           int* h_seq_order) {
    const int total = cula_kda_num_chunks(h_cu_seqlens, N);
    if (total < 0) return total;
    if (!h_chunk_indices || !h_chunk_offsets) return CULA_KDA_EINVAL;
    int c = 0;
    for (int n = 0; n < N; ++n) {
        h_chunk_offsets[n] = c;
        const int chunks = (h_cu_seqlens[n + 1] - h_cu_seqlens[n] + kda::BT - 1) / kda::BT;
        for (int i = 0; i < chunks; ++i, ++c) {
            h_chunk_indices[2 * c] = n;
            h_chunk_indices[2 * c + 1] = i;
        }
    }
    h_chunk_offsets[N] = c;
    if (h_seq_order) {            // longest sequence first, ties in input order (stable insertion sort: N is small)
        for (int n = 0; n < N; ++n) {
            const int len = h_cu_seqlens[n + 1] - h_cu_seqlens[n];
            int pos = n;
            while (pos > 0) {
                const int m = h_seq_order[pos - 1];
                if (h_cu_seqlens[m + 1] - h_cu_seqlens[m] >= len) break;
                h_seq_order[pos] = m;
                --pos;
            }
            h_seq_order[pos] = n;
        }
    }
    return 0;
}

extern "C" int cula_kda_bwd_scratch_floats(void) { return kda::BWD_SCRATCH_FLOATS; }

extern "C" int cula_kda_bwd_grad_scale(const void* d_do, long long n_do, const float* d_dht, long long n_dht,
                                       unsigned int* d_amax, float* d_gscale, void* stream) {
    if (!d_do || !d_amax || !d_gscale || n_do < 0 || n_dht < 0) return CULA_KDA_EINVAL;
    if (misaligned(d_do) || misaligned(d_dht)) return CULA_KDA_EALIGN;
    return kda_launch_grad_scale(d_do, (size_t)n_do, d_dht, (size_t)n_dht, d_amax, d_gscale, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_bwd_scan(const void* d_tiles, const void* d_do, const float* d_dht, const float* d_gscale,
                                 void* d_dvn_out, float* d_ds_out, float* d_dh0, const int* d_cu_seqlens,
                                 const int* d_chunk_offsets, const int* d_seq_order, int N, int T, int H, int* d_status,
                                 void* stream) {
    if (N == 0) return 0;
    if (!d_tiles || !d_do || !d_gscale || !d_status || N < 0 || H <= 0) return CULA_KDA_EINVAL;
    if ((d_dvn_out == nullptr) != (d_ds_out == nullptr)) return CULA_KDA_EINVAL;
    if (!d_dvn_out && !d_dh0) return CULA_KDA_EINVAL;     // nothing to produce
    if ((d_cu_seqlens == nullptr) != (d_chunk_offsets == nullptr)) return CULA_KDA_EINVAL;
    if (!d_cu_seqlens && T <= 0) return CULA_KDA_EINVAL;
    if (misaligned(d_tiles) || misaligned(d_do) || misaligned(d_dvn_out) || misaligned(d_ds_out)) return CULA_KDA_EALIGN;
    kda::BwdScanParams p{};
    p.tiles = static_cast<const unsigned char*>(d_tiles);
    p.d_o = d_do; p.dht = d_dht; p.gscale = d_gscale; p.dvn_out = d_dvn_out; p.ds_out = d_ds_out; p.dh0 = d_dh0;
    p.cu_seqlens = d_cu_seqlens; p.chunk_offsets = d_chunk_offsets; p.seq_order = d_seq_order;
    p.status = d_status; p.T = T; p.H = H; p.N = N;
    return kda_launch_bwd_scan(&p, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_bwd_dense(const float* d_h32, const float* d_ds, const void* d_vnew, const void* d_dvn,
                                  const void* d_do, const void* d_v, const void* d_beta, int beta_is_fp32,
                                  const float* d_akk, const float* d_gscale, void* d_dv, float* d_scratch,
                                  const int* d_cu_seqlens, const int* d_chunk_indices, int num_chunks, int T, int H,
                                  int* d_status, void* stream) {
    if (num_chunks == 0) return 0;
    if (!d_h32 || !d_ds || !d_vnew || !d_dvn || !d_do || !d_v || !d_beta || !d_akk || !d_gscale || !d_dv || !d_scratch || !d_status ||
        num_chunks < 0 || H <= 0)
        return CULA_KDA_EINVAL;
    if ((d_cu_seqlens == nullptr) != (d_chunk_indices == nullptr)) return CULA_KDA_EINVAL;
    if (!d_cu_seqlens && T <= 0) return CULA_KDA_EINVAL;
    if (misaligned(d_h32) || misaligned(d_ds) || misaligned(d_vnew) || misaligned(d_dvn) || misaligned(d_do) ||
        misaligned(d_v) || misaligned(d_akk) || misaligned(d_dv) || misaligned(d_scratch))
        return CULA_KDA_EALIGN;
    kda::BwdDenseParams p{};
    p.h32 = d_h32; p.ds = d_ds; p.vnew = d_vnew; p.dvn = d_dvn; p.d_o = d_do; p.v = d_v; p.beta = d_beta;
    p.akk = d_akk; p.gscale = d_gscale; p.dv = d_dv; p.scratch = d_scratch;
    p.cu_seqlens = d_cu_seqlens; p.chunk_indices = d_chunk_indices; p.T = T; p.H = H; p.status = d_status;
    p.beta_fp32 = beta_is_fp32 & CULA_KDA_BETA_FP32; p.beta_logit = (beta_is_fp32 & CULA_KDA_BETA_LOGIT) != 0;
    return kda_launch_bwd_dense(&p, num_chunks, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_bwd_gated(const void* d_q, const void* d_k, const void* d_g, int g_is_fp32, const void* d_beta,
                                  int beta_is_fp32, const float* d_A_log, const float* d_dt_bias, const float* d_akk,
                                  const float* d_mkk, const float* d_scratch, const float* d_gscale, void* d_dq, void* d_dk,
                                  void* d_dg, void* d_dbeta, float* d_dA_log, float* d_ddt_bias, const int* d_cu_seqlens,
                                  const int* d_chunk_indices, int num_chunks, int T, int H, float scale, int use_qk_l2norm,
                                  int gate_mode, float lower_bound, void* stream) {
    if (num_chunks == 0) return 0;
    if (!d_q || !d_k || !d_g || !d_beta || !d_akk || !d_mkk || !d_scratch || !d_gscale || !d_dq || !d_dk || !d_dg ||
        !d_dbeta || num_chunks < 0 || H <= 0)
        return CULA_KDA_EINVAL;
    if (gate_mode < 0 || gate_mode > 2 || (gate_mode != 0 && !d_A_log)) return CULA_KDA_EINVAL;
    if ((d_cu_seqlens == nullptr) != (d_chunk_indices == nullptr)) return CULA_KDA_EINVAL;
    if (!d_cu_seqlens && T <= 0) return CULA_KDA_EINVAL;
    const bool per_head = (g_is_fp32 & CULA_KDA_G_PER_HEAD) != 0;
    if (g_is_fp32 & ~(CULA_KDA_G_FP32 | CULA_KDA_G_PER_HEAD)) return CULA_KDA_EINVAL;
    if (misaligned(d_q) || misaligned(d_k) || misaligned(d_akk) || misaligned(d_mkk) || misaligned(d_scratch) || misaligned(d_dq) ||
        misaligned(d_dk) || (!per_head && (misaligned(d_g) || misaligned(d_dg))))
        return CULA_KDA_EALIGN;
    kda::BwdGatedParams p{};
    p.q = d_q; p.k = d_k; p.g = d_g; p.beta = d_beta; p.A_log = d_A_log; p.dt_bias = d_dt_bias; p.akk = d_akk;
    p.mkk = d_mkk; p.scratch = d_scratch; p.gscale = d_gscale; p.dq = d_dq; p.dk = d_dk; p.dg = d_dg; p.dbeta = d_dbeta;
    p.dA_log = d_dA_log; p.ddt_bias = d_ddt_bias; p.cu_seqlens = d_cu_seqlens; p.chunk_indices = d_chunk_indices;
    p.T = T; p.H = H; p.g_fp32 = g_is_fp32 & CULA_KDA_G_FP32; p.g_per_head = per_head;
    p.beta_fp32 = beta_is_fp32 & CULA_KDA_BETA_FP32; p.beta_logit = (beta_is_fp32 & CULA_KDA_BETA_LOGIT) != 0;
    p.use_l2norm = use_qk_l2norm; p.gate_mode = gate_mode; p.lower_bound = lower_bound; p.scale = scale;
    return kda_launch_bwd_gated(&p, num_chunks, static_cast<cudaStream_t>(stream));
}

extern "C" int kda_launch_gate(const kda::GateArgs* a, int backward, cudaStream_t stream);
extern "C" int kda_launch_beta_sigmoid(const void* x, int x_fp32, const float* dy, void* out, long long n, int backward,
                                       cudaStream_t stream);

extern "C" int cula_kda_gate_fwd(const void* d_g, int g_is_fp32, const float* d_A_log, const float* d_dt_bias, void* d_y,
                                 int y_is_fp32, long long M, int H, int K, int use_lower_bound, float lower_bound, void* stream) {
    if (M == 0) return 0;
    if (!d_g || !d_A_log || !d_y || M < 0 || H <= 0 || K < 32 || K % 8 != 0) return CULA_KDA_EINVAL;
    if (misaligned(d_g) || misaligned(d_y)) return CULA_KDA_EALIGN;
    kda::GateArgs a{d_g, d_A_log, d_dt_bias, nullptr, d_y, nullptr, nullptr, M, H, K, g_is_fp32, y_is_fp32, 0, use_lower_bound, lower_bound};
    return kda_launch_gate(&a, 0, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_gate_bwd(const void* d_g, int g_is_fp32, const float* d_A_log, const float* d_dt_bias, const void* d_dy,
                                 int dy_is_fp32, void* d_dg, float* d_dA_log, float* d_ddt_bias, long long M, int H, int K,
                                 int use_lower_bound, float lower_bound, void* stream) {
    if (M == 0) return 0;
    if (!d_g || !d_A_log || !d_dy || !d_dg || M < 0 || H <= 0 || K < 32 || K % 8 != 0) return CULA_KDA_EINVAL;
    if (misaligned(d_g) || misaligned(d_dy) || misaligned(d_dg)) return CULA_KDA_EALIGN;
    kda::GateArgs a{d_g, d_A_log, d_dt_bias, d_dy, d_dg, d_dA_log, d_ddt_bias, M, H, K, g_is_fp32, 0, dy_is_fp32, use_lower_bound, lower_bound};
    return kda_launch_gate(&a, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_beta_sigmoid_fwd(const void* d_x, int x_is_fp32, float* d_y, long long n, void* stream) {
    if (n == 0) return 0;
    if (!d_x || !d_y || n < 0) return CULA_KDA_EINVAL;
    return kda_launch_beta_sigmoid(d_x, x_is_fp32, nullptr, d_y, n, 0, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_beta_sigmoid_bwd(const void* d_x, int x_is_fp32, const float* d_dy, void* d_dx, long long n, void* stream) {
    if (n == 0) return 0;
    if (!d_x || !d_dy || !d_dx || n < 0) return CULA_KDA_EINVAL;
    return kda_launch_beta_sigmoid(d_x, x_is_fp32, d_dy, d_dx, n, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int kda_launch_short_conv(const kda::ConvArgs* a, int num_chunks, int backward, cudaStream_t stream);
extern "C" int kda_launch_rms_norm_gated(const kda::NormArgs* a, int backward, cudaStream_t stream);

extern "C" int cula_kda_short_conv_fwd(const void* d_x, const float* d_w, const float* d_bias, const float* d_cache_in, void* d_y,
                                       float* d_cache_out, const int* d_cu_seqlens, const int* d_chunk_indices,
                                       int num_chunks, int T, int D, int W, int use_silu, void* stream) {
    if (num_chunks == 0) return 0;
    if (!d_x || !d_w || !d_y || num_chunks < 0 || D <= 0 || D % 8 != 0 || W < 1 || W > 4) return CULA_KDA_EINVAL;
    if ((d_cu_seqlens == nullptr) != (d_chunk_indices == nullptr)) return CULA_KDA_EINVAL;
    if (!d_cu_seqlens && T <= 0) return CULA_KDA_EINVAL;
    if (misaligned(d_x) || misaligned(d_y)) return CULA_KDA_EALIGN;
    kda::ConvArgs a{};
    a.x = static_cast<const __nv_bfloat16*>(d_x); a.w = d_w; a.bias = d_bias; a.cache_in = d_cache_in;
    a.y = static_cast<__nv_bfloat16*>(d_y); a.cache_out = d_cache_out; a.cu_seqlens = d_cu_seqlens; a.chunk_indices = d_chunk_indices;
    a.T = T; a.D = D; a.W = W; a.silu = use_silu;
    return kda_launch_short_conv(&a, num_chunks, 0, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_short_conv_bwd(const void* d_x, const float* d_w, const float* d_bias, const float* d_cache_in,
                                       const void* d_dy, void* d_dx, float* d_dw, float* d_dbias, const int* d_cu_seqlens,
                                       const int* d_chunk_indices, int num_chunks, int T, int D, int W, int use_silu, void* stream) {
    if (num_chunks == 0) return 0;
    if (!d_x || !d_w || !d_dy || !d_dx || !d_dw || num_chunks < 0 || D <= 0 || D % 8 != 0 || W < 1 || W > 4) return CULA_KDA_EINVAL;
    if ((d_cu_seqlens == nullptr) != (d_chunk_indices == nullptr)) return CULA_KDA_EINVAL;
    if (!d_cu_seqlens && T <= 0) return CULA_KDA_EINVAL;
    if (misaligned(d_x) || misaligned(d_dy) || misaligned(d_dx)) return CULA_KDA_EALIGN;
    kda::ConvArgs a{};
    a.x = static_cast<const __nv_bfloat16*>(d_x); a.w = d_w; a.bias = d_bias; a.cache_in = d_cache_in;
    a.dy = static_cast<const __nv_bfloat16*>(d_dy); a.dx = static_cast<__nv_bfloat16*>(d_dx); a.dw = d_dw; a.dbias = d_dbias;
    a.cu_seqlens = d_cu_seqlens; a.chunk_indices = d_chunk_indices; a.T = T; a.D = D; a.W = W; a.silu = use_silu;
    return kda_launch_short_conv(&a, num_chunks, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int cula_kda_rms_norm_gated_fwd(const void* d_x, const void* d_g, const float* d_w, void* d_y, float* d_rstd,
                                           long long R, int D, int use_swish, float eps, void* stream) {
    if (R == 0) return 0;
    if (!d_x || !d_g || !d_w || !d_y || !d_rstd || R < 0 || !(D == 128 || D == 256 || D == 512 || D == 1024)) return CULA_KDA_EINVAL;
    if (misaligned(d_x) || misaligned(d_g) || misaligned(d_y)) return CULA_KDA_EALIGN;
    kda::NormArgs a{};
    a.x = static_cast<const __nv_bfloat16*>(d_x); a.g = static_cast<const __nv_bfloat16*>(d_g); a.w = d_w;
    a.y = static_cast<__nv_bfloat16*>(d_y); a.rstd = d_rstd; a.R = R; a.D = D; a.swish = use_swish; a.eps = eps;
    const int rc = kda_launch_rms_norm_gated(&a, 0, static_cast<cudaStream_t>(stream));
    return rc == -1 ? CULA_KDA_EINVAL : rc;
}

extern "C" int cula_kda_rms_norm_gated_bwd(const void* d_x, const void* d_g, const float* d_w, const float* d_rstd,
                                           const void* d_dy, void* d_dx, void* d_dg, float* d_dw, long long R, int D,
                                           int use_swish, void* stream) {
    if (R == 0) return 0;
    if (!d_x || !d_g || !d_w || !d_rstd || !d_dy || !d_dx || !d_dg || !d_dw || R < 0 ||
        !(D == 128 || D == 256 || D == 512 || D == 1024))
        return CULA_KDA_EINVAL;
    if (misaligned(d_x) || misaligned(d_g) || misaligned(d_dy) || misaligned(d_dx) || misaligned(d_dg)) return CULA_KDA_EALIGN;
    kda::NormArgs a{};
    a.x = static_cast<const __nv_bfloat16*>(d_x); a.g = static_cast<const __nv_bfloat16*>(d_g); a.w = d_w;
    a.rstd = const_cast<float*>(d_rstd); a.dy = static_cast<const __nv_bfloat16*>(d_dy); a.dx = static_cast<__nv_bfloat16*>(d_dx);
    a.dg = static_cast<__nv_bfloat16*>(d_dg); a.dw = d_dw; a.R = R; a.D = D; a.swish = use_swish;
    const int rc = kda_launch_rms_norm_gated(&a, 1, static_cast<cudaStream_t>(stream));
    return rc == -1 ? CULA_KDA_EINVAL : rc;
}

extern "C" int kda_launch_selftest_wait(int* status, int limit, cudaStream_t stream);

extern "C" int cula_kda_selftest_bounded_wait(int* d_status, int max_polls, void* stream) {
    if (!d_status || max_polls <= 0 || max_polls > (1 << 22)) return CULA_KDA_EINVAL;
    return kda_launch_selftest_wait(d_status, max_polls, static_cast<cudaStream_t>(stream));
}

extern "C" const char* cula_kda_strerror(int code) {
    if (code == 0) return "ok";
    if (code == CULA_KDA_EINVAL) return "invalid argument (null pointer, non-positive size or bad enum)";
    if (code == CULA_KDA_EALIGN) return "pointer is not 16-byte aligned";
    if (code == CULA_KDA_ETOOBIG) return "num_chunks * H exceeds the fixed capacity of cula_kda_fwd_noalloc (256 tiles)";
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown error";
}
