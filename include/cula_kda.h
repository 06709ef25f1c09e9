/*
 * C ABI of libcula_kda.so: the B200 (sm_100a) kernels behind cula.kda.chunk_kda.
 *
 * Conventions
 *   - every pointer named d_* is a DEVICE pointer owned by the caller; the library never allocates,
 *     frees or keeps device memory (same ownership rule as the reference's native layer, where
 *     Python allocates every output and workspace: cula/kda/chunk_intra.py:776-791,
 *     cula/ops/chunk_delta_h.py:2119-2138);
 *   - tensors are contiguous, token-major: q/k/g [B*T, H, 128], v/o [B*T, H, 128], beta [B*T, H];
 *     a packed (varlen) batch is one sequence axis of cu_seqlens[N] tokens, B == 1;
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, nothing synchronises;
 *   - return value: 0 = ok, < 0 = argument error (CULA_KDA_E*), > 0 = a cudaError_t from the launch.
 *     The reference instead throws c10::Error from TORCH_CHECK (csrc/api/kda_sm100.cu:46-50) and
 *     exit(1)s on CUDA errors (csrc/kerutils/include/kerutils/common/common.h:24-31).
 *   - head dim is 128 for keys and values, chunk length 64 (cula/kda/chunk.py:54,386-388).
 */
#ifndef CULA_KDA_H_
#define CULA_KDA_H_

#ifdef __cplusplus
extern "C" {
#endif

#define CULA_KDA_EINVAL (-1)   /* null pointer / non-positive size / bad enum */
#define CULA_KDA_EALIGN (-2)   /* a pointer is not 16-byte aligned */
#define CULA_KDA_ETOOBIG (-3)  /* problem exceeds the fixed capacity of cula_kda_fwd_noalloc */

#define CULA_KDA_NOALLOC_MAX_TILES 256   /* capacity of cula_kda_fwd_noalloc: num_chunks * H */

/* bits of the g_is_fp32 argument: element type and layout of the gate tensor (and of its gradient) */
#define CULA_KDA_G_FP32 1       /* fp32 elements (bf16 otherwise) */
#define CULA_KDA_G_PER_HEAD 2   /* [B*T, H]: one gate per (token, head) shared by all 128 key channels -- the scalar-gate
                                   (gated delta rule, "GDN") variant of the same pipeline; [B*T, H, 128] otherwise */

/* bits of the beta_is_fp32 argument */
#define CULA_KDA_BETA_FP32 1    /* fp32 elements (bf16 otherwise) */
#define CULA_KDA_BETA_LOGIT 2   /* beta holds raw logits: sigmoid is applied in-kernel, and the backward pass returns the
                                   gradient w.r.t. the logits (fuses fused_beta_sigmoid, fla/ops/kda/gate.py:431) */

#define CULA_KDA_GATE_NONE 0         /* g already holds the natural-log decay (use_gate_in_kernel=False) */
#define CULA_KDA_GATE_SOFTPLUS 1     /* a = -exp(A_log[h]) * softplus(g + dt_bias[h,:]) */
#define CULA_KDA_GATE_LOWER_BOUND 2  /* a = lower_bound * sigmoid(exp(A_log[h]) * (g + dt_bias[h,:])) (safe_gate) */

/* Bytes of one forward tile pack, the per-(chunk, head) record handed from the chunk-parallel stage
 * to the state scan: w, qg, kg, Aqk, u (fp16), 2^g_last (fp32), pre-swizzled for the scan. */
int cula_kda_tile_pack_bytes(void);

/* Shared memory (bytes) each kernel asks for; lets a caller check the device limit up front. */
int cula_kda_fwd_intra_smem_bytes(void);
int cula_kda_fwd_scan_smem_bytes(void);

/*
 * Chunk-parallel forward stage, one CTA per (chunk, head).
 * Replaces, fused into one launch:
 *   l2norm_fwd(q), l2norm_fwd(k)            cula/kda/chunk.py:58-60
 *   kda_gate_chunk_cumsum / chunk_local_cumsum   cula/kda/chunk_fwd.py:69-80
 *   chunk_kda_fwd_intra_cuda(q,k,g,beta,cu_seqlens,chunk_indices,Aqk_out,Akk_out,tile_counter,scale,
 *                            chunk_size,use_tf32_inverse,unified_gref)   csrc/api/pybind.cu:70-79, csrc/api/kda_sm100.cu:22-68
 *   recompute_w_u_cuda(k,v,beta,A,g,cu_seqlens,chunk_indices,w_out,u_out,kg_out,chunk_size,q,qg_out)
 *                                                                 csrc/api/kda_sm100.cu:70-120
 * d_cu_seqlens [N+1] / d_chunk_indices [num_chunks][2] (sequence, chunk-in-sequence) are the tables of
 * prepare_chunk_indices; pass both NULL for a fixed-length batch of sequences of T tokens.
 * d_tiles: num_chunks*H tile packs (output). d_akk: optional [num_chunks*H][64][64] fp32 (I+L)^-1;
 * d_mkk: optional [num_chunks*H][64][64] fp32 strictly-lower gated k k^T Gram matrix (both kept for backward).
 * d_status: one int the kernel sets non-zero if a bounded wait on a tensor-core completion barrier gave up.
 */
int cula_kda_fwd_intra(const void* d_q, const void* d_k, const void* d_v,
                       const void* d_g, int g_is_fp32,
                       const void* d_beta, int beta_is_fp32,
                       const float* d_A_log, const float* d_dt_bias,
                       const int* d_cu_seqlens, const int* d_chunk_indices,
                       int num_chunks, int T, int H,
                       float scale, int use_qk_l2norm, int gate_mode, float lower_bound,
                       void* d_tiles, float* d_akk, float* d_mkk, int* d_status, void* stream);

/*
 * Sequential state scan fused with the output stage, one CTA per (sequence, head, value half).
 * Replaces chunk_gated_delta_rule_fwd_h(k=kg, w, u, gk, initial_state, output_final_state, cu_seqlens, ...)
 *   (cula/ops/chunk_delta_h.py:1991-2168, called at cula/kda/chunk_fwd.py:111-120) and
 *   chunk_gla_fwd_o(q, v_new, g, A=Aqk, h, o, scale, ...) (cula/ops/fwd_o.py:1755-1852, chunk_fwd.py:131-143).
 * d_h0 / d_ht: [N, H, 128, 128] fp32 or NULL. d_o: [B*T, H, 128] bf16; only rows of real tokens are written
 * (d_o may be NULL when d_vnew_out is given: the backward recomputation needs the states, not the output).
 * d_h_out (bf16 [num_chunks*H][128][128], state entering each chunk) and d_vnew_out (fp16
 * [num_chunks*H][64][128]) and d_h32_out (the same states in fp32, for the backward pass) are optional;
 * d_vnew_out must be given whenever a state output is.
 * d_chunk_offsets [N+1]: first global chunk of each sequence (prepare_chunk_offsets);
 * d_seq_order [N]: optional launch order of the sequences (longest first balances a ragged batch).
 * d_status: one int the kernel sets non-zero if a bounded pipeline wait gave up (never in a healthy run).
 */
int cula_kda_fwd_scan(const void* d_tiles, const float* d_h0, void* d_o, float* d_ht,
                      void* d_h_out, void* d_vnew_out, float* d_h32_out,
                      const int* d_cu_seqlens, const int* d_chunk_offsets, const int* d_seq_order,
                      int N, int T, int H, int* d_status, void* stream);

/*
 * Index tables of a packed batch, computed on the host from HOST memory (h_*): what prepare_chunk_indices
 * (fla/ops/utils/index.py:138-149) and prepare_chunk_offsets_i32 (cula/ops/chunk_delta_h.py:42-47) produce with torch.
 * cula_kda_num_chunks: sum of ceil(len / 64) over the N sequences (< 0 on a bad cu_seqlens).
 * cula_kda_build_chunk_tables: h_chunk_indices [num_chunks][2] (sequence, chunk in sequence), h_chunk_offsets [N+1]
 * (first global chunk of every sequence), h_seq_order [N] or NULL (sequences by decreasing length, the launch order
 * cula_kda_fwd_scan balances a ragged batch with). The caller copies them to the device.
 */
int cula_kda_num_chunks(const int* h_cu_seqlens, int N);
int cula_kda_build_chunk_tables(const int* h_cu_seqlens, int N, int* h_chunk_indices, int* h_chunk_offsets,
                                int* h_seq_order);

/* ------------------------------------------------------------------------------------------------------------
 * Backward pass. The reference's backward is all Triton / flash-linear-attention kernels plus a recompute of
 * its forward intermediates (cula/kda/chunk_bwd.py:432-604); here it is four launches after re-running the two
 * forward launches with d_akk, d_mkk, d_h32_out and d_vnew_out set.
 * All gradient-like intermediates are carried in units of a power-of-two scale s (d_gscale = {s, 1/s}).
 * ------------------------------------------------------------------------------------------------------------ */

/* floats per (chunk, head) of the scratch record passed from cula_kda_bwd_dense to cula_kda_bwd_gated */
int cula_kda_bwd_scratch_floats(void);

/* s = 2^k with max(|dO|, |dht|) * s in [4, 8). d_amax: one uint32 of workspace. No counterpart in the reference
 * (its bf16 intermediates need no range management; ours are fp16). */
int cula_kda_bwd_grad_scale(const void* d_do, long long n_do, const float* d_dht, long long n_dht,
                            unsigned int* d_amax, float* d_gscale, void* stream);

/* Reverse state scan: d_dvn_out (fp16 [num_chunks*H][64][128], gradient w.r.t. v_new), d_ds_out (fp32
 * [num_chunks*H][128][128], gradient w.r.t. the state leaving each chunk), d_dh0 ([N,H,128,128] fp32 or NULL).
 * d_dvn_out and d_ds_out may both be NULL when only d_dh0 is wanted (first pass of the context-parallel backward).
 * Replaces chunk_gated_delta_rule_bwd_dhu (fla/ops/common/chunk_delta_h.py:659-718, cula/kda/chunk_bwd.py:541-555)
 * and the dv half of chunk_kda_bwd_dAv (cula/kda/chunk_bwd.py:510-520). */
int cula_kda_bwd_scan(const void* d_tiles, const void* d_do, const float* d_dht, const float* d_gscale,
                      void* d_dvn_out, float* d_ds_out, float* d_dh0,
                      const int* d_cu_seqlens, const int* d_chunk_offsets, const int* d_seq_order,
                      int N, int T, int H, int* d_status, void* stream);

/* Chunk-parallel dense products with the carried states (tcgen05 tensor cores; the fp32 states arrive through TMA
 * tensor maps built per call from d_h32 / d_ds); writes d_dv (bf16, final) and the scratch record. d_status: device
 * status word of the bounded waits. Replaces the state-dependent half of chunk_kda_bwd_wy_dqkg_fused (cula/kda/chunk_bwd.py:557-574) and the dAqk
 * half of chunk_kda_bwd_dAv. */
int cula_kda_bwd_dense(const float* d_h32, const float* d_ds, const void* d_vnew, const void* d_dvn,
                       const void* d_do, const void* d_v, const void* d_beta, int beta_is_fp32,
                       const float* d_akk, const float* d_gscale, void* d_dv, float* d_scratch,
                       const int* d_cu_seqlens, const int* d_chunk_indices, int num_chunks, int T, int H, int* d_status,
                       void* stream);

/* Chunk-parallel gated part: Akk / Gram-matrix VJPs, reverse cumulative sum, gate and L2-norm VJPs.
 * Writes d_dq, d_dk (bf16), d_dg (dtype of g), d_dbeta (dtype of beta); accumulates d_dA_log [H] and
 * d_ddt_bias [H*128] with atomics (caller zeroes them). Replaces the rest of chunk_kda_bwd_wy_dqkg_fused,
 * chunk_kda_bwd_intra (cula/kda/chunk_intra.py:796-860), chunk_local_cumsum(reverse) + kda_gate_bwd
 * (cula/kda/chunk_bwd.py:594-602) and l2norm_bwd (cula/kda/chunk.py:190-192). */
int cula_kda_bwd_gated(const void* d_q, const void* d_k, const void* d_g, int g_is_fp32,
                       const void* d_beta, int beta_is_fp32, const float* d_A_log, const float* d_dt_bias,
                       const float* d_akk, const float* d_mkk, const float* d_scratch, const float* d_gscale,
                       void* d_dq, void* d_dk, void* d_dg, void* d_dbeta, float* d_dA_log, float* d_ddt_bias,
                       const int* d_cu_seqlens, const int* d_chunk_indices, int num_chunks, int T, int H,
                       float scale, int use_qk_l2norm, int gate_mode, float lower_bound, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * Context parallelism (one long sequence split into contiguous shards, one per GPU). The reference reaches this
 * through flash-linear-attention's cp_context (cula/kda/chunk_fwd.py:99-109,122-127; fla/ops/cp/chunk_delta_h.py).
 * A shard acts on the carried state as S_out = M S_in + C.
 * ------------------------------------------------------------------------------------------------------------ */

/* Per (sequence, head): d_c_out [N,H,128,128] = final state of the shard started from zero, d_m_out [N,H,128,128] =
 * transition matrix. Same tile packs and tables as cula_kda_fwd_scan. Replaces
 * chunk_gated_delta_rule_fwd_h_pre_process (fla/ops/cp/chunk_delta_h.py:736-795). */
int cula_kda_cp_transition(const void* d_tiles, float* d_c_out, float* d_m_out,
                           const int* d_cu_seqlens, const int* d_chunk_offsets, int N, int T, int H,
                           int* d_status, void* stream);

/* d_s_out [H,128,128] = S after  S <- d_h0 (zero when NULL);  for j in [0, n): S <- M_j S + C_j,  where element j of
 * the chain sits at d_c_all + j * stride_floats and d_m_all + j * stride_floats ([H,128,128] fp32 each, in this GPU's
 * own memory: gathered transitions or the rank's own). stride_floats <= 0 means densely packed (H*128*128).
 * d_c_all == NULL stands for C_j = 0 (product of the M_j: composing the transitions of a shard's segments).
 * Replaces the merge step (fla/ops/cp/chunk_delta_h.py:797-817). */
int cula_kda_cp_fold(const float* d_c_all, const float* d_m_all, const float* d_h0, float* d_s_out, int n, int H,
                     long long stride_floats, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * Decode: one token per sequence against a pool of fp32 states, updated in place (the step after prefill).
 * Replaces the compiled CuTe-DSL callable behind kda_decode / fused_sigmoid_gating_delta_rule_update
 * (cula/ops/kda_decode.py:1794-2096; kernel arguments at :2080-2094):
 *   gate = exp(-exp(A_log[hv]) * softplus(a + dt_bias[hv,:])), v_new = sigmoid(b) (v - S^T (gate k)),
 *   S <- diag(gate) S + k v_new^T, o = S^T (scale q), with q, k L2-normalised when use_qk_l2norm != 0.
 * d_q, d_k [N,H,128] bf16; d_v, d_o [N,HV,V] bf16 (V % 32 == 0); d_a [N,HV,128] and d_b [N,HV] bf16 or fp32;
 * d_A_log [HV]; d_dt_bias [HV,128] or NULL; d_state [pool_size,HV,V,128] (state_is_kv == 0, the reference's "vk"
 * default) or [pool_size,HV,128,V] (state_is_kv != 0); d_state_indices [N] int32 pool slots or NULL (slot = n).
 * A negative slot skips the sequence (no state access, its output row is zeroed); a slot >= pool_size sets *d_status to 2
 * and touches nothing. HV must be a multiple of H (grouped value heads).
 * ------------------------------------------------------------------------------------------------------------ */
int cula_kda_decode(const void* d_q, const void* d_k, const void* d_v, const void* d_a, int a_is_fp32,
                    const void* d_b, int b_is_fp32, const float* d_A_log, const float* d_dt_bias,
                    float* d_state, const int* d_state_indices, void* d_o, int N, int H, int HV, int V,
                    int pool_size, float scale, int use_qk_l2norm, float softplus_beta,
                    float softplus_threshold, int state_is_kv, int* d_status, void* stream);

/*
 * Whole forward pass (both launches above) for callers that cannot allocate device memory themselves -- a runtime
 * that has given all device memory to its own pool, a plugin inside a foreign memory manager, a path where
 * cudaMalloc's device-wide synchronisation is unacceptable. It has no counterpart in the reference, whose Python
 * layer allocates every workspace with torch. The tile packs live in a fixed 18.1 MiB array inside the library's
 * device image (held by every GPU that loads the library until the process exits), so:
 *   - num_chunks * H must not exceed CULA_KDA_NOALLOC_MAX_TILES (= 256), else CULA_KDA_ETOOBIG is returned;
 *   - all calls on a device share that array: calls that can overlap on the GPU race, serialise them;
 *   - the first call on a device resolves the array's address; make it before any stream capture on that device.
 * Arguments as in cula_kda_fwd_intra / cula_kda_fwd_scan (d_chunk_offsets/d_chunk_indices/d_cu_seqlens all NULL for
 * a fixed-length batch, where num_chunks must equal N * ceil(T/64)). Never calls cudaMalloc or cudaFree.
 */
int cula_kda_noalloc_max_tiles(void);
int cula_kda_fwd_noalloc(const void* d_q, const void* d_k, const void* d_v, const void* d_g, int g_is_fp32,
                         const void* d_beta, int beta_is_fp32, const float* d_A_log, const float* d_dt_bias,
                         const float* d_h0, void* d_o, float* d_ht,
                         const int* d_cu_seqlens, const int* d_chunk_indices, const int* d_chunk_offsets,
                         int num_chunks, int N, int T, int H,
                         float scale, int use_qk_l2norm, int gate_mode, float lower_bound,
                         int* d_status, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * Layer-side elementwise operators next to chunk_kda (for callers that do not let chunk_kda activate the gate itself).
 * Replace flash-linear-attention's fused_kda_gate (KDAGateFunction, fla/ops/kda/gate.py:282-345; kernels :88-279) and
 * fused_beta_sigmoid (fla/ops/kda/gate.py:348-432), which callers of the reference use around cula.kda.chunk_kda.
 * d_g, d_y, d_dy, d_dg: [M, H, K] (M tokens), K a multiple of 8 and >= 32; bf16 or fp32 as flagged.
 *   use_lower_bound == 0:  y = -exp(A_log[h]) * softplus(g + dt_bias[h,:])
 *   use_lower_bound != 0:  y = lower_bound * sigmoid(exp(A_log[h]) * (g + dt_bias[h,:]))
 * Backward writes d_dg in the dtype of g and ACCUMULATES d_dA_log [H] and d_ddt_bias [H*K] (either may be NULL) with
 * atomics: the caller zeroes them first.
 * ------------------------------------------------------------------------------------------------------------ */
int cula_kda_gate_fwd(const void* d_g, int g_is_fp32, const float* d_A_log, const float* d_dt_bias, void* d_y,
                      int y_is_fp32, long long M, int H, int K, int use_lower_bound, float lower_bound, void* stream);
int cula_kda_gate_bwd(const void* d_g, int g_is_fp32, const float* d_A_log, const float* d_dt_bias, const void* d_dy,
                      int dy_is_fp32, void* d_dg, float* d_dA_log, float* d_ddt_bias, long long M, int H, int K,
                      int use_lower_bound, float lower_bound, void* stream);
/* y = sigmoid(x) in fp32 over n elements (x bf16 or fp32); backward: dx = dy * y * (1 - y) in the dtype of x. */
int cula_kda_beta_sigmoid_fwd(const void* d_x, int x_is_fp32, float* d_y, long long n, void* stream);
int cula_kda_beta_sigmoid_bwd(const void* d_x, int x_is_fp32, const float* d_dy, void* d_dx, long long n, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * The two layer operators on either side of chunk_kda in a Kimi-Linear block (fla/layers/kda.py:147-165, 191, 306).
 *
 * Short causal depthwise convolution (+ SiLU) of the q / k / v projections; replaces ShortConvolution / causal_conv1d
 * (fla/modules/convolution.py: causal_conv1d(x, weight, bias, residual, initial_state, output_final_state,
 * activation, cu_seqlens, ...)). d_x, d_y, d_dy, d_dx: [tokens, D] bf16 (D % 8 == 0); d_w [D, W] fp32, W <= 4, tap
 * W-1 multiplies the current token; d_bias [D] or NULL; d_cache_in / d_cache_out [N, D, W] fp32 or NULL: the last W
 * inputs of every sequence, newest last (what a decode step continues from). Same packed-batch tables as the
 * attention kernels (NULL, NULL for a fixed-length batch of sequences of T tokens); num_chunks as there.
 * Backward ACCUMULATES d_dw [D, W] and d_dbias [D] (may be NULL) with atomics: the caller zeroes them.
 *
 * Gated RMS norm of the attention output; replaces FusedRMSNormGated / rms_norm_gated
 * (fla/modules/fused_norm_gate.py:846-869): y = x * rsqrt(mean(x^2) + eps) * w * act(g), act = sigmoid
 * (use_swish == 0) or g * sigmoid(g). Rows of D in {128, 256, 512, 1024} bf16; d_rstd [R] fp32 is written by the
 * forward pass and read by the backward pass, which ACCUMULATES d_dw [D] with atomics.
 * ------------------------------------------------------------------------------------------------------------ */
int cula_kda_short_conv_fwd(const void* d_x, const float* d_w, const float* d_bias, const float* d_cache_in, void* d_y,
                            float* d_cache_out, const int* d_cu_seqlens, const int* d_chunk_indices,
                            int num_chunks, int T, int D, int W, int use_silu, void* stream);
int cula_kda_short_conv_bwd(const void* d_x, const float* d_w, const float* d_bias, const float* d_cache_in,
                            const void* d_dy, void* d_dx, float* d_dw, float* d_dbias, const int* d_cu_seqlens,
                            const int* d_chunk_indices, int num_chunks, int T, int D, int W, int use_silu, void* stream);
int cula_kda_rms_norm_gated_fwd(const void* d_x, const void* d_g, const float* d_w, void* d_y, float* d_rstd,
                                long long R, int D, int use_swish, float eps, void* stream);
int cula_kda_rms_norm_gated_bwd(const void* d_x, const void* d_g, const float* d_w, const float* d_rstd,
                                const void* d_dy, void* d_dx, void* d_dg, float* d_dw, long long R, int D,
                                int use_swish, void* stream);

/*
 * Self-test of the bounded waits: launches one warp that waits on a barrier nothing completes; after max_polls
 * polls (1 .. 2^22) the wait gives up, *d_status is set to 1 (the time-out status every kernel above reports through
 * its d_status argument) and the kernel returns. Lets a deployment check that a stuck pipeline ends in a status
 * word instead of a hung GPU. No counterpart in the reference: its device waits are unbounded
 * (cula/ops/chunk_delta_h.py:1303-1424 pipeline waits) and its CUDA errors end the process
 * (csrc/kerutils/include/kerutils/common/common.h:24-31).
 * Status word values: 0 ok, 1 a bounded wait timed out, 2 state-pool index out of range (decode),
 * 3 a forward intermediate (w, u) left the fp16 range or is not finite.
 */
int cula_kda_selftest_bounded_wait(int* d_status, int max_polls, void* stream);

/* Human-readable text for a return value of the functions above. */
const char* cula_kda_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif /* CULA_KDA_H_ */
