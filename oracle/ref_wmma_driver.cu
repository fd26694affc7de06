// Times the REFERENCE's own WMMA kernels, recompiled for sm_100a from the reference tree where it
// lies (the .cu file is included, never copied; its main() is renamed away). TEST / BASELINE
// INFRASTRUCTURE: built by oracle/Makefile (target wmma) into oracle/_ref/, used only as a
// reported baseline ("the existing kernel on the same GPU"), never by the library.
//
//   REF_VARIANT 0: gemm_shmem_tc_async           (matmul_shmem_tc_async.cu:494-557)
//   REF_VARIANT 2: gemm_shmem_tc_async_opt_port  (matmul_shmem_tc_async_opt_port_2.cu:1088-1168)
//
// usage: ref_wmma_<variant> M tile_dim segment_dim_k tile_group_m num_stages producers consumers reps
//        [bar_steps_a bar_steps_b bar_step_rows_a bar_step_rows_b]      (square problem M = N = K)
#define main reference_main_not_used
#if REF_VARIANT == 0
#include "matmul_shmem_tc_async.cu"
#else
#include "matmul_shmem_tc_async_opt_port_2.cu"
#endif
#undef main

#include <cstdlib>
#include <vector>

int main(int argc, char **argv) {
    if (argc < 9) {
        printf("usage: %s M tile seg_k group_m stages producers consumers reps [bsa bsb bsra bsrb]\n", argv[0]);
        return 2;
    }
    const int M = atoi(argv[1]), tile = atoi(argv[2]), seg = atoi(argv[3]), group_m = atoi(argv[4]);
    const int stages = atoi(argv[5]), P = atoi(argv[6]), C = atoi(argv[7]), reps = atoi(argv[8]);
    const int bsa = argc > 9 ? atoi(argv[9]) : 0, bsb = argc > 10 ? atoi(argv[10]) : 0;
    const int bsra = argc > 11 ? atoi(argv[11]) : tile, bsrb = argc > 12 ? atoi(argv[12]) : tile;
    (void)group_m; (void)bsa; (void)bsb; (void)bsra; (void)bsrb;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, 0) != cudaSuccess) { printf("{\"error\": \"no device\"}\n"); return 1; }
    const size_t n = size_t(M) * M;
    std::vector<half> hA(n), hB(n);
    uint32_t x = 12345u;
    for (size_t i = 0; i < n; ++i) {
        x = x * 1664525u + 1013904223u; hA[i] = __float2half(((x >> 8) & 0xFFFF) / 32768.0f - 1.0f);
        x = x * 1664525u + 1013904223u; hB[i] = __float2half(((x >> 8) & 0xFFFF) / 32768.0f - 1.0f);
    }
    half *A, *B; float *Cm, *D;
    cudaMalloc(&A, n * 2); cudaMalloc(&B, n * 2); cudaMalloc(&Cm, n * 4); cudaMalloc(&D, n * 4);
    cudaMemcpy(A, hA.data(), n * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(B, hB.data(), n * 2, cudaMemcpyHostToDevice);
    cudaMemset(Cm, 0, n * 4); cudaMemset(D, 0, n * 4);
    auto launch = [&]() {
#if REF_VARIANT == 0
        gemm_shmem_tc_async<half, float>(A, B, Cm, D, 1.0f, 0.0f, M, M, M, tile, seg, stages, P, C, prop.multiProcessorCount);
#else
        gemm_shmem_tc_async_opt_port<half, float>(A, B, Cm, D, 1.0f, 0.0f, M, M, M, tile, seg, bsa, bsb, bsra, bsrb, group_m,
                                                  stages, P, C, prop.multiProcessorCount);
#endif
    };
    launch();
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("{\"error\": \"%s\"}\n", cudaGetErrorString(e)); return 1; }
    cudaEvent_t t0, t1; cudaEventCreate(&t0); cudaEventCreate(&t1);
    cudaEventRecord(t0);
    for (int i = 0; i < reps; ++i) launch();
    cudaEventRecord(t1); cudaEventSynchronize(t1);
    float ms = 0; cudaEventElapsedTime(&ms, t0, t1);
    e = cudaGetLastError();
    // spot check: 64 elements against the reference's own host arithmetic (matmul_test.h:316-320)
    std::vector<float> hD(size_t(M) * 64);
    cudaMemcpy(hD.data(), D, hD.size() * 4, cudaMemcpyDeviceToHost);
    float maxerr = 0;
    for (int j = 0; j < 64; ++j) {
        float acc = 0;
        for (int k = 0; k < M; ++k) acc += __half2float(hA[k]) * __half2float(hB[size_t(j) * M + k]);
        maxerr = fmaxf(maxerr, fabsf(acc - hD[j]));
    }
    printf("{\"kernel\": \"reference_wmma_v%d\", \"M\": %d, \"tile\": %d, \"seg_k\": %d, \"stages\": %d, \"P\": %d, \"C\": %d, "
           "\"ms\": %.4f, \"tflops\": %.2f, \"spot_maxerr\": %.4g, \"cuda\": \"%s\"}\n",
           REF_VARIANT, M, tile, seg, stages, P, C, ms / reps, 2.0 * M * double(M) * M * 1e-12 / (ms / reps * 1e-3), maxerr,
           cudaGetErrorString(e));
    return 0;
}
