/*
 * CPU oracle (plain C) for the chunk_kda forward path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may load this library.
 *
 * It restates the fp32 token recurrence the reference's tests compare against
 * (flash-linear-attention 0.5.1, un-vendored dependency of the reference:
 *  fla/ops/kda/naive.py:45-66 for the recurrence, fla/ops/kda/gate.py:26-54 and :57-69 for the
 *  two gate activations; called by the reference at tests/test_kda.py:106-114 and :259-267),
 * with the L2 normalisation of tests/test_kda.py:107-108 (x / max(||x||, 1e-12)).
 *
 * Parity pin: tests/test_oracle.py runs this against the stored outputs of the third-party
 * functions themselves (tests/golden/, made by tests/golden/make_golden.py).
 *
 * Per (sequence n, head h), state S[K][V]:
 *     S <- diag(exp(a_t)) S ;  r = v_t - S^T k_t ;  S <- S + (beta_t k_t) r^T ;  o_t = S^T (scale q_t)
 *
 * Build:  gcc -O3 -march=native -fopenmp -shared -fPIC oracle/naive_kda.c -o oracle/libnaive_kda.so -lm
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

/* gate_mode: 0 = g already holds the log decay; 1 = softplus form; 2 = lower-bound sigmoid form. */
static float gate_act(float graw, float alpha, float bias, int gate_mode, float lower_bound) {
    if (gate_mode == 0) return graw;
    float x = graw + bias;
    if (gate_mode == 2) return lower_bound / (1.f + expf(-alpha * x));
    return -alpha * softplus_f(x);
}

int naive_kda_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Set the number of OpenMP threads of later calls (a launcher may have exported OMP_NUM_THREADS=1). */
void naive_kda_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/*
 * q,k,g: [total_T, H, K]   v,o: [total_T, H, V]   beta: [total_T, H]   (all fp32, token-major)
 * cu_seqlens: [N+1] token offsets of the N sequences (a fixed-length batch passes 0,T,2T,...)
 * A_log [H], dt_bias [H*K] (may be NULL), h0 [N,H,K,V] (may be NULL), ht [N,H,K,V] (may be NULL)
 * Returns 0, or -1 on a bad argument.
 */
int naive_kda_fwd(const float* q, const float* k, const float* v, const float* g, const float* beta,
                  const float* A_log, const float* dt_bias, const float* h0,
                  float* o, float* ht, const int* cu_seqlens,
                  int N, int H, int K, int V, float scale,
                  int use_l2norm, int gate_mode, float lower_bound) {
    if (!q || !k || !v || !g || !beta || !o || !cu_seqlens || N < 0 || H <= 0 || K <= 0 || V <= 0) return -1;
    if (gate_mode != 0 && !A_log) return -1;
    int fail = 0;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int n = 0; n < N; ++n) {
        for (int h = 0; h < H; ++h) {
            float* S = (float*)malloc(sizeof(float) * (size_t)K * V);
            float* kn = (float*)malloc(sizeof(float) * K);
            float* qn = (float*)malloc(sizeof(float) * K);
            float* r = (float*)malloc(sizeof(float) * V);
            if (!S || !kn || !qn || !r) { fail = 1; free(S); free(kn); free(qn); free(r); continue; }
            if (h0) memcpy(S, h0 + ((size_t)n * H + h) * K * V, sizeof(float) * (size_t)K * V);
            else memset(S, 0, sizeof(float) * (size_t)K * V);
            float alpha = gate_mode ? expf(A_log[h]) : 0.f;
            for (int t = cu_seqlens[n]; t < cu_seqlens[n + 1]; ++t) {
                const float* qt = q + ((size_t)t * H + h) * K;
                const float* kt = k + ((size_t)t * H + h) * K;
                const float* gt = g + ((size_t)t * H + h) * K;
                const float* vt = v + ((size_t)t * H + h) * V;
                float* ot = o + ((size_t)t * H + h) * V;
                float bt = beta[(size_t)t * H + h];
                float qs = 1.f, ks = 1.f;
                if (use_l2norm) {
                    float sq = 0.f, sk = 0.f;
                    for (int d = 0; d < K; ++d) { sq += qt[d] * qt[d]; sk += kt[d] * kt[d]; }
                    qs = 1.f / fmaxf(sqrtf(sq), 1e-12f);
                    ks = 1.f / fmaxf(sqrtf(sk), 1e-12f);
                }
                for (int d = 0; d < K; ++d) { qn[d] = qt[d] * qs * scale; kn[d] = kt[d] * ks; }
                for (int j = 0; j < V; ++j) r[j] = 0.f;
                for (int d = 0; d < K; ++d) {           /* decay, and accumulate S^T k */
                    float a = gate_act(gt[d], alpha, dt_bias ? dt_bias[h * K + d] : 0.f, gate_mode, lower_bound);
                    float e = expf(a), kd = kn[d];
                    float* Sd = S + (size_t)d * V;
                    for (int j = 0; j < V; ++j) { Sd[j] *= e; r[j] += kd * Sd[j]; }
                }
                for (int j = 0; j < V; ++j) { r[j] = vt[j] - r[j]; ot[j] = 0.f; }
                for (int d = 0; d < K; ++d) {           /* rank-1 update, and read-out */
                    float bk = bt * kn[d], qd = qn[d];
                    float* Sd = S + (size_t)d * V;
                    for (int j = 0; j < V; ++j) { Sd[j] += bk * r[j]; ot[j] += qd * Sd[j]; }
                }
            }
            if (ht) memcpy(ht + ((size_t)n * H + h) * K * V, S, sizeof(float) * (size_t)K * V);
            free(S); free(kn); free(qn); free(r);
        }
    }
    return fail ? -1 : 0;
}
