// Plain launch-parameter structs shared between the C-ABI layer and the kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kda {

enum GateMode : int {
    GATE_NONE = 0,         // g already holds the natural-log decay
    GATE_SOFTPLUS = 1,     // a = -exp(A_log[h]) * softplus(g + dt_bias[h,:])
    GATE_LOWER_BOUND = 2,  // a = lower_bound * sigmoid(exp(A_log[h]) * (g + dt_bias[h,:]))
};

struct IntraParams {
    const void* q;            // [B*T, H, 128] bf16
    const void* k;            // [B*T, H, 128] bf16
    const void* v;            // [B*T, H, 128] bf16
    const void* g;            // [B*T, H, 128] bf16 or fp32 ([B*T, H] when g_per_head)
    const void* beta;         // [B*T, H] bf16 or fp32
    const float* A_log;       // [H] or null
    const float* dt_bias;     // [H*128] or null
    const int* cu_seqlens;    // [N+1] or null (fixed length)
    const int* chunk_indices; // [NT][2] or null (fixed length)
    unsigned char* tiles;     // [NT*H] tile packs
    float* akk_out;           // [NT*H][64][64] fp32 or null
    float* mkk_out;           // [NT*H][64][64] fp32 strict-lower gated k k^T Gram matrix, or null
    int* status;              // device status word
    int T;                    // tokens per sequence when cu_seqlens is null
    int H;
    int num_tiles;            // num_chunks * H (filled in by the launcher)
    int g_fp32;
    int g_per_head;           // 1: g is [B*T, H], one gate per (token, head) shared by all 128 channels (scalar-gate variant)
    int beta_fp32;
    int beta_logit;           // 1: beta holds the raw logits; sigmoid is applied in-kernel
    int use_l2norm;
    int gate_mode;
    float lower_bound;
    float scale;
};

struct ScanParams {
    const unsigned char* tiles;   // [NT*H] tile packs
    const float* h0;              // [N, H, 128, 128] fp32 or null
    void* o;                      // [B*T, H, 128] bf16
    float* ht;                    // [N, H, 128, 128] fp32 or null
    void* h_out;                  // per-chunk incoming state, bf16, or null
    float* h32_out;               // per-chunk incoming state, fp32, or null
    float* m_out;                 // [N, H, 128, 128] shard transition matrices (transition launch only)
    void* vnew_out;               // per-chunk v_new, fp16, or null
    const int* cu_seqlens;        // [N+1] or null
    const int* chunk_offsets;     // [N+1] first global chunk of each sequence, or null
    const int* seq_order;         // [N] launch order (longest first) or null
    int* status;                  // device status word
    int T;
    int H;
    int N;                        // number of sequences
    int group_major;              // transition launch only: grid is (head, sequence, column group) instead of
                                  // (column group, head, sequence); set by the launcher
};

struct BwdScanParams {
    const unsigned char* tiles;   // [NT*H] forward tile packs
    const void* d_o;              // [B*T, H, 128] bf16 upstream gradient
    const float* dht;             // [N, H, 128, 128] fp32 or null
    const float* gscale;          // device: {s, 1/s}; all gradient-like operands are carried in units of s
    void* dvn_out;                // [NT*H][64][128] fp16, gradient w.r.t. v_new (units of s)
    float* ds_out;                // [NT*H][128][128] fp32, gradient w.r.t. the state leaving each chunk (units of s)
    float* dh0;                   // [N, H, 128, 128] fp32 or null (true units)
    const int* cu_seqlens;
    const int* chunk_offsets;
    const int* seq_order;
    int* status;
    int T;
    int H;
    int N;
};

// fp32 scratch record written per (chunk, head) by the dense backward stage, read by the gated stage
constexpr int SCR_DQG = 0;            // [64][128] gradient w.r.t. qg = scale q 2^g
constexpr int SCR_DW = 8192;          // [64][128] gradient w.r.t. w
constexpr int SCR_DKG = 16384;        // [64][128] gradient w.r.t. kg
constexpr int SCR_DPS = 24576;        // [64][64]  gradient w.r.t. Aqk (lower triangle incl. diagonal)
constexpr int SCR_DAU = 28672;        // [64][64]  stril(dVn (beta V)^T): the u-part of the gradient w.r.t. Akk
constexpr int SCR_DBU = 32768;        // [64]      rowsum(Zu * V)
constexpr int SCR_DD = 32832;         // [128]     sum_v S dS'
constexpr int BWD_SCRATCH_FLOATS = 32960;

struct BwdDenseParams {
    const float* h32;             // [NT*H][128][128] state entering each chunk
    const float* ds;              // [NT*H][128][128] gradient w.r.t. the state leaving each chunk (units of s)
    const void* vnew;             // [NT*H][64][128] fp16
    const void* dvn;              // [NT*H][64][128] fp16 (units of s)
    const void* d_o;              // [B*T, H, 128] bf16
    const void* v;                // [B*T, H, 128] bf16
    const void* beta;
    const float* akk;             // [NT*H][64][64] fp32
    const float* gscale;
    void* dv;                     // [B*T, H, 128] bf16 (output)
    float* scratch;               // [NT*H][BWD_SCRATCH_FLOATS]
    const int* cu_seqlens;
    const int* chunk_indices;
    int T;
    int H;
    int beta_fp32;
    int beta_logit;               // 1: beta holds the raw logits
    int* status;                  // device status word (bounded waits)
};

struct BwdGatedParams {
    const void* q;
    const void* k;
    const void* g;
    const void* beta;
    const float* A_log;
    const float* dt_bias;
    const float* akk;             // [NT*H][64][64] fp32
    const float* mkk;             // [NT*H][64][64] fp32: strict-lower sum_d k_i k_j 2^(g_i-g_j)
    const float* scratch;         // [NT*H][BWD_SCRATCH_FLOATS]
    const float* gscale;
    void* dq;                     // [B*T, H, 128] bf16
    void* dk;                     // [B*T, H, 128] bf16
    void* dg;                     // [B*T, H, 128] dtype of g
    void* dbeta;                  // [B*T, H] dtype of beta
    float* dA_log;                // [H] fp32, accumulated with atomics (zero it first) or null
    float* ddt_bias;              // [H*128] fp32, accumulated with atomics, or null
    const int* cu_seqlens;
    const int* chunk_indices;
    int T;
    int H;
    int g_fp32;
    int g_per_head;               // 1: g and dg are [B*T, H] (one gate per token and head)
    int beta_fp32;
    int beta_logit;               // 1: beta holds the raw logits; dbeta is then the gradient w.r.t. the logits
    int use_l2norm;
    int gate_mode;
    float lower_bound;
    float scale;
};

// short causal depthwise convolution (forward and backward)
struct ConvArgs {
    const __nv_bfloat16* x;       // [Ttot, D]
    const float* w;               // [D, W]
    const float* bias;            // [D] or null
    const float* cache_in;        // [N, D, W] or null
    __nv_bfloat16* y;             // [Ttot, D]            (forward)
    float* cache_out;             // [N, D, W] or null    (forward)
    const __nv_bfloat16* dy;      // [Ttot, D]            (backward)
    __nv_bfloat16* dx;            // [Ttot, D]            (backward)
    float* dw;                    // [D, W] accumulated with atomics (backward)
    float* dbias;                 // [D] accumulated with atomics, or null
    const int* cu_seqlens;        // [N+1] or null
    const int* chunk_indices;     // [NT][2] or null
    int T, D, W, silu;
};

// gated RMS norm (forward and backward)
struct NormArgs {
    const __nv_bfloat16* x;   // [R, D]
    const __nv_bfloat16* g;   // [R, D]
    const float* w;           // [D]
    __nv_bfloat16* y;         // [R, D]          (forward)
    float* rstd;              // [R]             (forward: written; backward: read)
    const __nv_bfloat16* dy;  // [R, D]          (backward)
    __nv_bfloat16* dx;        // [R, D]
    __nv_bfloat16* dg;        // [R, D]
    float* dw;                // [D] accumulated with atomics
    long long R;
    int D, swish;
    float eps;
};

// stand-alone gate activation (forward and backward)
struct GateArgs {
    const void* g;        // [M, H*K] bf16 or fp32
    const float* A_log;   // [H]
    const float* dt_bias; // [H*K] or null
    const void* dy;       // [M, H*K] gradient w.r.t. the output (backward), bf16 or fp32
    void* out;            // forward: y; backward: dg (dtype of g)
    float* dA_log;        // [H] (backward, accumulated with atomics; zero it first) or null
    float* ddt_bias;      // [H*K] (backward, accumulated with atomics) or null
    long long M;          // tokens
    int H, K;
    int g_fp32, out_fp32, dy_fp32;
    int use_lower_bound;
    float lower_bound;
};

}  // namespace kda
