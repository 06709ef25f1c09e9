// Plain launch-parameter structs shared between the C-ABI layer and the kernels.
#pragma once
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
    const void* g;            // [B*T, H, 128] bf16 or fp32
    const void* beta;         // [B*T, H] bf16 or fp32
    const float* A_log;       // [H] or null
    const float* dt_bias;     // [H*128] or null
    const int* cu_seqlens;    // [N+1] or null (fixed length)
    const int* chunk_indices; // [NT][2] or null (fixed length)
    unsigned char* tiles;     // [NT*H] tile packs
    float* akk_out;           // [NT*H][64][64] fp32 or null
    int* status;              // device status word
    int T;                    // tokens per sequence when cu_seqlens is null
    int H;
    int num_tiles;            // num_chunks * H (filled in by the launcher)
    int g_fp32;
    int beta_fp32;
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
    void* vnew_out;               // per-chunk v_new, fp16, or null
    const int* cu_seqlens;        // [N+1] or null
    const int* chunk_offsets;     // [N+1] first global chunk of each sequence, or null
    const int* seq_order;         // [N] launch order (longest first) or null
    int* status;                  // device status word
    int T;
    int H;
    int N;                        // number of sequences
};

}  // namespace kda
