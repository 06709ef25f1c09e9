/* A host program in plain C that runs the chunk_kda forward through the C ABI alone (no Python, no torch): it is what
 * a non-Python runtime would write. Reads raw tensors from a directory, allocates device memory with the CUDA runtime,
 * calls cula_kda_fwd_intra + cula_kda_fwd_scan, writes o and the final state back as raw files.
 *
 *   forward_from_c <dir> <B> <T> <H>
 *   inputs  (little-endian raw): q.bin k.bin v.bin g.bin (bf16 [B,T,H,128]), beta.bin (bf16 [B,T,H]),
 *                                A_log.bin (f32 [H]), dt_bias.bin (f32 [H*128]), h0.bin (f32 [B,H,128,128])
 *            optional cu_seqlens.bin (int32 [N+1]): a packed batch of N sequences (then B must be 1, h0 is [N,H,128,128]);
 *            the index tables are built with cula_kda_build_chunk_tables
 *   outputs: o.bin (bf16 [B,T,H,128]), ht.bin (f32 [B or N,H,128,128])
 * Gate: lower_bound * sigmoid(exp(A_log) (g + dt_bias)) with lower_bound = -5, L2-normalised q / k, scale 128^-0.5.
 */
#include <cuda_runtime_api.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "cula_kda.h"

#define CHECK_CUDA(x)                                                                  \
    do {                                                                               \
        cudaError_t e_ = (x);                                                          \
        if (e_ != cudaSuccess) {                                                       \
            fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));                   \
            return 2;                                                                  \
        }                                                                              \
    } while (0)
#define CHECK_KDA(x)                                                                   \
    do {                                                                               \
        int r_ = (x);                                                                  \
        if (r_ != 0) {                                                                 \
            fprintf(stderr, "%s: %d (%s)\n", #x, r_, cula_kda_strerror(r_));           \
            return 3;                                                                  \
        }                                                                              \
    } while (0)

static void* load_to_device(const char* dir, const char* name, size_t bytes) {
    char path[1024];
    snprintf(path, sizeof path, "%s/%s", dir, name);
    FILE* f = fopen(path, "rb");
    if (!f) return NULL;
    void* host = malloc(bytes);
    size_t got = fread(host, 1, bytes, f);
    fclose(f);
    void* dev = NULL;
    if (got != bytes || cudaMalloc(&dev, bytes) != cudaSuccess ||
        cudaMemcpy(dev, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess)
        dev = NULL;
    free(host);
    return dev;
}

static int store_from_device(const char* dir, const char* name, const void* dev, size_t bytes) {
    char path[1024];
    snprintf(path, sizeof path, "%s/%s", dir, name);
    void* host = malloc(bytes);
    int ok = cudaMemcpy(host, dev, bytes, cudaMemcpyDeviceToHost) == cudaSuccess;
    FILE* f = ok ? fopen(path, "wb") : NULL;
    ok = f && fwrite(host, 1, bytes, f) == bytes;
    if (f) fclose(f);
    free(host);
    return ok ? 0 : 1;
}

int main(int argc, char** argv) {
    if (argc != 5) {
        fprintf(stderr, "usage: %s <dir> <B> <T> <H>\n", argv[0]);
        return 1;
    }
    const char* dir = argv[1];
    const int B = atoi(argv[2]), T = atoi(argv[3]), H = atoi(argv[4]);
    const size_t th = (size_t)B * T * H;
    int num_chunks = B * ((T + 63) / 64), N = B;
    int *d_cu = NULL, *d_idx = NULL, *d_off = NULL, *d_order = NULL;
    {   /* packed batch? */
        char path[1024];
        snprintf(path, sizeof path, "%s/cu_seqlens.bin", dir);
        FILE* f = fopen(path, "rb");
        if (f) {
            int cu[1025];
            const int count = (int)fread(cu, sizeof(int), 1025, f);
            fclose(f);
            N = count - 1;
            num_chunks = cula_kda_num_chunks(cu, N);
            if (B != 1 || N < 1 || num_chunks < 0) {
                fprintf(stderr, "bad packed batch\n");
                return 1;
            }
            int* idx = (int*)malloc(sizeof(int) * 2 * (size_t)(num_chunks > 0 ? num_chunks : 1));
            int* off = (int*)malloc(sizeof(int) * (size_t)(N + 1));
            int* order = (int*)malloc(sizeof(int) * (size_t)N);
            CHECK_KDA(cula_kda_build_chunk_tables(cu, N, idx, off, order));
            CHECK_CUDA(cudaMalloc((void**)&d_cu, sizeof(int) * (N + 1)));
            CHECK_CUDA(cudaMalloc((void**)&d_idx, sizeof(int) * 2 * (num_chunks > 0 ? num_chunks : 1)));
            CHECK_CUDA(cudaMalloc((void**)&d_off, sizeof(int) * (N + 1)));
            CHECK_CUDA(cudaMalloc((void**)&d_order, sizeof(int) * N));
            CHECK_CUDA(cudaMemcpy(d_cu, cu, sizeof(int) * (N + 1), cudaMemcpyHostToDevice));
            CHECK_CUDA(cudaMemcpy(d_idx, idx, sizeof(int) * 2 * num_chunks, cudaMemcpyHostToDevice));
            CHECK_CUDA(cudaMemcpy(d_off, off, sizeof(int) * (N + 1), cudaMemcpyHostToDevice));
            CHECK_CUDA(cudaMemcpy(d_order, order, sizeof(int) * N, cudaMemcpyHostToDevice));
            free(idx); free(off); free(order);
        }
    }
    const size_t state_bytes = (size_t)N * H * 128 * 128 * 4;

    void* q = load_to_device(dir, "q.bin", th * 128 * 2);
    void* k = load_to_device(dir, "k.bin", th * 128 * 2);
    void* v = load_to_device(dir, "v.bin", th * 128 * 2);
    void* g = load_to_device(dir, "g.bin", th * 128 * 2);
    void* beta = load_to_device(dir, "beta.bin", th * 2);
    float* A_log = (float*)load_to_device(dir, "A_log.bin", (size_t)H * 4);
    float* dt_bias = (float*)load_to_device(dir, "dt_bias.bin", (size_t)H * 128 * 4);
    float* h0 = (float*)load_to_device(dir, "h0.bin", state_bytes);
    if (!q || !k || !v || !g || !beta || !A_log || !dt_bias || !h0) {
        fprintf(stderr, "could not load the inputs from %s\n", dir);
        return 1;
    }
    void *tiles = NULL, *o = NULL;
    float* ht = NULL;
    int* status = NULL;
    CHECK_CUDA(cudaMalloc(&tiles, (size_t)num_chunks * H * cula_kda_tile_pack_bytes()));
    CHECK_CUDA(cudaMalloc(&o, th * 128 * 2));
    CHECK_CUDA(cudaMemset(o, 0, th * 128 * 2));
    CHECK_CUDA(cudaMalloc((void**)&ht, state_bytes));
    CHECK_CUDA(cudaMalloc((void**)&status, sizeof(int)));
    CHECK_CUDA(cudaMemset(status, 0, sizeof(int)));
    cudaStream_t stream;
    CHECK_CUDA(cudaStreamCreate(&stream));

    CHECK_KDA(cula_kda_fwd_intra(q, k, v, g, 0, beta, 0, A_log, dt_bias, d_cu, d_idx, num_chunks, T, H, 0.08838834764831845f,
                                 1, CULA_KDA_GATE_LOWER_BOUND, -5.0f, tiles, NULL, NULL, status, stream));
    CHECK_KDA(cula_kda_fwd_scan(tiles, h0, o, ht, NULL, NULL, NULL, d_cu, d_off, d_order, N, T, H, status, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    int host_status = -1;
    CHECK_CUDA(cudaMemcpy(&host_status, status, sizeof(int), cudaMemcpyDeviceToHost));
    if (host_status != 0) {
        fprintf(stderr, "kernel status %d\n", host_status);
        return 4;
    }
    /* argument errors come back as codes, nothing is thrown and nothing exits */
    if (cula_kda_fwd_scan(NULL, h0, o, ht, NULL, NULL, NULL, NULL, NULL, NULL, B, T, H, status, stream) != CULA_KDA_EINVAL) return 5;
    if (cula_kda_fwd_intra((const char*)q + 2, k, v, g, 0, beta, 0, A_log, dt_bias, NULL, NULL, num_chunks, T, H, 1.0f, 1,
                           CULA_KDA_GATE_LOWER_BOUND, -5.0f, tiles, NULL, NULL, status, stream) != CULA_KDA_EALIGN)
        return 6;
    if (store_from_device(dir, "o.bin", o, th * 128 * 2) || store_from_device(dir, "ht.bin", ht, state_bytes)) return 7;
    printf("C_HOST_OK\n");
    return 0;
}
