// The reference's three test families, re-targeted at the B200 launchers (include/b200_matmul.h):
//
//   correctness  constant matrices A = 1, B = 10, C = 1, closed-form expectation, atol 1e-3, random
//                tile-multiple square dims up to the maximum  (RunCorrectnessTestSquare,
//                matmul_shmem_tc_async_opt_port_2.cu:1170-1278; matmul_test.h:227-232, :279-288)
//   accuracy     seeded U[-1,1) A, B^T, C, full CPU recompute in the reference's arithmetic,
//                count of elements outside atol 0.1  (RunAccuracyTestSquare, :1280-1390)
//   performance  1 warm-up + num_reps timed launches between CUDA events, 2*M*N*K/t TFLOPS
//                (RunPerformanceTestSquare, :1392-1499)
//
// swept over the same tunables and the same three barrier granularities (:1213-1232). Inputs are
// seeded (the reference seeds from the clock). TEST INFRASTRUCTURE: the CPU recompute is the
// oracle (oracle/gemm_oracle.c); the launchers under test never touch it.
//
// usage: b200_matmul_test <correctness|accuracy|performance> [dim] [quick]
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "b200_matmul.h"

extern "C" {
int oracle_gemm(const uint16_t *A, const uint16_t *Bt, const float *C, float *D, float alpha, float beta, int64_t M,
                int64_t N, int64_t K, int dtype, int num_threads);
float oracle_constant_expected(float a, float b, float c, float alpha, float beta, int64_t K);
int64_t oracle_count_incorrect(const float *expected, const float *got, int64_t count, float atol);
}

using namespace b200_matmul;

static const int WMMA_M = 16, WMMA_N = 16;  // the granularity unit of the reference's sweeps

#define CHECK(x)                                                                  \
    do {                                                                          \
        cudaError_t e_ = (x);                                                     \
        if (e_ != cudaSuccess) {                                                  \
            printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
            exit(3);                                                              \
        }                                                                         \
    } while (0)

struct Fixture {  // the role of MatmulTestGemmSquare (matmul_test.h:187-225), seeded
    int dim_max, tile_dim;
    std::vector<uint16_t> a, b;
    std::vector<float> c, res;
    uint64_t rng;
    Fixture(int dim_max_, int tile_dim_, bool constant, uint64_t seed)
        : dim_max(dim_max_), tile_dim(tile_dim_), a(size_t(dim_max_) * dim_max_), b(a.size()), c(a.size()), res(a.size()),
          rng(seed * 0x9E3779B97F4A7C15ull + 1) {
        if (constant) {
            for (size_t i = 0; i < a.size(); ++i) { a[i] = 0x3C00; b[i] = 0x4900; c[i] = 1.0f; }  // 1, 10, 1
        } else {
            b200_fill_u16_host(a.data(), 0, a.size(), seed, 1, 0, 1.0f, B200_F16);
            b200_fill_u16_host(b.data(), 0, b.size(), seed, 2, 0, 1.0f, B200_F16);
            b200_fill_f32_host(c.data(), 0, c.size(), seed, 3, 0, 1.0f);
        }
    }
    int next_dim() {  // GetMatDim (matmul_test.h:263-268) with a seeded generator
        rng = rng * 6364136223846793005ull + 1442695040888963407ull;
        int dim = int((rng >> 33) % uint64_t(dim_max + 1));
        return dim <= tile_dim ? tile_dim : dim - dim % tile_dim;
    }
};

struct Sweep {
    int tile_lo, tile_hi, seg_lo, seg_hi, group_lo, group_hi, stages_lo, stages_hi, p_lo, p_hi, c_lo, c_hi;
};

template <typename F>
static void for_each_config(const Sweep &s, int K, F f) {
    cudaDeviceProp prop;
    CHECK(cudaGetDeviceProperties(&prop, 0));
    for (int tile = s.tile_lo; tile <= s.tile_hi; tile *= 2)
        for (int seg = s.seg_lo; seg <= s.seg_hi; seg *= 2)
            for (int group = s.group_lo; group <= s.group_hi; ++group)
                for (int stages = s.stages_lo; stages <= s.stages_hi; ++stages)
                    for (int P = s.p_lo; P <= s.p_hi; P *= 2)
                        for (int C = s.c_lo; C <= s.c_hi; C *= 2) {
                            const int wtr = get_warp_tile_rows(tile, C), wtc = get_num_acc(tile, C) / wtr;
                            const int rows_a[3] = {WMMA_M, wtr * WMMA_M, tile}, rows_b[3] = {WMMA_N, wtc * WMMA_N, tile};
                            const int end_a[3] = {wtr - 1, tile / (wtr * WMMA_M), 0}, end_b[3] = {wtc - 1, tile / (wtc * WMMA_N), 0};
                            for (int i = 0; i < 3; ++i)
                                for (int bsa = 0; bsa <= end_a[i]; ++bsa)
                                    for (int bsb = 0; bsb <= end_b[i]; ++bsb) {
                                        // the harness's own filter (port_2.cu:1229-1232): fits shared memory, K splits
                                        if (get_shmem_req(tile, seg, bsa, bsb, rows_a[i], rows_b[i], stages, C) < 0 || K % seg) continue;
                                        f(tile, seg, bsa, bsb, rows_a[i], rows_b[i], group, stages, P, C, prop.multiProcessorCount);
                                    }
                        }
}

static int run_correctness(int dim_max, const Sweep &s, int num_reps, float alpha, float beta, float atol) {
    const size_t n = size_t(dim_max) * dim_max;
    half *A, *B; float *C, *D;
    CHECK(cudaMalloc(&A, n * 2)); CHECK(cudaMalloc(&B, n * 2)); CHECK(cudaMalloc(&C, n * 4)); CHECK(cudaMalloc(&D, n * 4));
    int failed = 0, total = 0;
    for (int tile = s.tile_lo; tile <= s.tile_hi; tile *= 2) {
        Fixture mt(dim_max, tile, true, 100 + tile);
        CHECK(cudaMemcpy(A, mt.a.data(), n * 2, cudaMemcpyHostToDevice));
        CHECK(cudaMemcpy(B, mt.b.data(), n * 2, cudaMemcpyHostToDevice));
        CHECK(cudaMemcpy(C, mt.c.data(), n * 4, cudaMemcpyHostToDevice));
        Sweep one = s; one.tile_lo = one.tile_hi = tile;
        for_each_config(one, dim_max, [&](int t, int seg, int bsa, int bsb, int ra, int rb, int group, int stages, int P, int Cw, int sms) {
            bool res = true;
            const int reps = seg <= t ? num_reps : 1;
            for (int j = 0; j < reps; ++j) {
                const int dim = seg <= t ? mt.next_dim() : dim_max;  // port_2.cu:1234 vs :1249
                CHECK(cudaMemset(D, 0, size_t(dim) * dim * 4));
                const int st = gemm_shmem_tc_async_opt_port<half, float>(A, B, C, D, alpha, beta, dim, dim, dim, t, seg, bsa, bsb, ra, rb,
                                                                         group, stages, P, Cw, sms);
                if (st != B200_OK) { res = false; printf("  status %d (%s)\n", st, b200_status_string(st)); break; }
                CHECK(cudaMemcpy(mt.res.data(), D, size_t(dim) * dim * 4, cudaMemcpyDeviceToHost));
                const float want = oracle_constant_expected(1.0f, 10.0f, 1.0f, alpha, beta, dim);
                for (size_t e = 0; e < size_t(dim) * dim && res; ++e)
                    if (!(fabsf(want - mt.res[e]) <= atol)) res = false;
            }
            ++total;
            if (!res) {
                ++failed;
                printf("(%d, %d, %d, %d, %d, %d, %d, %d, %d, %d): failed\n", t, seg, bsa, bsb, ra, rb, group, stages, P, Cw);
            }
        });
    }
    int info[4];
    const int dev = b200_device_status(nullptr, info);
    printf("correctness: %d configurations, %d failed, device status %d\n", total, failed, dev);
    cudaFree(A); cudaFree(B); cudaFree(C); cudaFree(D);
    return failed == 0 && dev == B200_OK ? 0 : 1;
}

static int run_accuracy(int dim, const Sweep &s, float alpha, float beta, float atol) {
    const size_t n = size_t(dim) * dim;
    half *A, *B; float *C, *D;
    CHECK(cudaMalloc(&A, n * 2)); CHECK(cudaMalloc(&B, n * 2)); CHECK(cudaMalloc(&C, n * 4)); CHECK(cudaMalloc(&D, n * 4));
    long long bad_total = 0; int total = 0, errors = 0;
    Fixture mt(dim, 128, false, 200 + dim);
    std::vector<float> want(n);
    oracle_gemm(mt.a.data(), mt.b.data(), mt.c.data(), want.data(), alpha, beta, dim, dim, dim, 0, 0);
    CHECK(cudaMemcpy(A, mt.a.data(), n * 2, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(B, mt.b.data(), n * 2, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(C, mt.c.data(), n * 4, cudaMemcpyHostToDevice));
    for_each_config(s, dim, [&](int t, int seg, int bsa, int bsb, int ra, int rb, int group, int stages, int P, int Cw, int sms) {
        CHECK(cudaMemset(D, 0, n * 4));
        const int st = gemm_shmem_tc_async_opt_port<half, float>(A, B, C, D, alpha, beta, dim, dim, dim, t, seg, bsa, bsb, ra, rb, group,
                                                                 stages, P, Cw, sms);
        ++total;
        if (st != B200_OK) { ++errors; printf("  status %d\n", st); return; }
        CHECK(cudaMemcpy(mt.res.data(), D, n * 4, cudaMemcpyDeviceToHost));
        const long long bad = oracle_count_incorrect(want.data(), mt.res.data(), (int64_t)n, atol);  // GetNumIncorrect's count
        bad_total += bad;
        if (bad) printf("(%d, %d, %d, %d, %d, %d, %d, %d, %d, %d): %lld / %zu outside atol\n", t, seg, bsa, bsb, ra, rb, group, stages, P, Cw, bad, n);
    });
    printf("accuracy %d^3: %d configurations, %lld elements outside atol %.3g, %d launch errors\n", dim, total, bad_total, atol, errors);
    cudaFree(A); cudaFree(B); cudaFree(C); cudaFree(D);
    return bad_total == 0 && errors == 0 ? 0 : 1;
}

static int run_performance(int dim, int num_reps) {
    const size_t n = size_t(dim) * dim;
    half *A, *B; float *C, *D;
    CHECK(cudaMalloc(&A, n * 2)); CHECK(cudaMalloc(&B, n * 2)); CHECK(cudaMalloc(&C, n * 4)); CHECK(cudaMalloc(&D, n * 4));
    CHECK(b200_fill_u16_device(A, 0, n, 5, 1, 0, 1.0f, B200_F16, nullptr) == 0 ? cudaSuccess : cudaErrorUnknown);
    CHECK(b200_fill_u16_device(B, 0, n, 5, 2, 0, 1.0f, B200_F16, nullptr) == 0 ? cudaSuccess : cudaErrorUnknown);
    CHECK(b200_fill_f32_device(C, 0, n, 5, 3, 0, 1.0f, nullptr) == 0 ? cudaSuccess : cudaErrorUnknown);
    cudaEvent_t start, stop;
    CHECK(cudaEventCreate(&start)); CHECK(cudaEventCreate(&stop));
    Sweep s = {128, 128, 64, 128, 8, 8, 3, 4, 1, 2, 4, 4};
    cudaDeviceProp prop; CHECK(cudaGetDeviceProperties(&prop, 0));
    for (int seg = s.seg_lo; seg <= s.seg_hi; seg *= 2)
        for (int stages = s.stages_lo; stages <= s.stages_hi; ++stages)
            for (int P = s.p_lo; P <= s.p_hi; P *= 2) {
                if (get_shmem_req(128, seg, 0, 0, 128, 128, stages, 4) < 0) continue;
                auto launch = [&]() { return gemm_shmem_tc_async_opt_port<half, float>(A, B, C, D, 1.0f, 1.0f, dim, dim, dim, 128, seg, 8, stages, P, 4, prop.multiProcessorCount); };
                if (launch() != B200_OK) continue;
                CHECK(cudaEventRecord(start, 0));
                for (int j = 0; j < num_reps; ++j) launch();
                CHECK(cudaEventRecord(stop, 0));
                CHECK(cudaEventSynchronize(stop));
                float ms = 0; CHECK(cudaEventElapsedTime(&ms, start, stop));
                printf("(128, %d, %d, %d, %d, 4): %.2f TFLOPS\n", seg, 8, stages, P, 2.0 * dim * 1e-9 * dim * dim * num_reps / ms);
            }
    cudaFree(A); cudaFree(B); cudaFree(C); cudaFree(D);
    return 0;
}

// The reference instantiates every launcher for <half, half> as well (matmul_shmem_tc_async.cu:411-478): fp16 C and
// D, half scalars. Constant matrices at sizes whose result is exact in fp16 (10 * dim + 1 <= 2048).
static int run_half_output(int dim_max) {
    const size_t n = size_t(dim_max) * dim_max;
    half *A, *B, *C, *D;
    CHECK(cudaMalloc(&A, n * 2)); CHECK(cudaMalloc(&B, n * 2)); CHECK(cudaMalloc(&C, n * 2)); CHECK(cudaMalloc(&D, n * 2));
    std::vector<half> a(n, __float2half(1.0f)), b(n, __float2half(10.0f)), c(n, __float2half(1.0f)), res(n);
    CHECK(cudaMemcpy(A, a.data(), n * 2, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(B, b.data(), n * 2, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(C, c.data(), n * 2, cudaMemcpyHostToDevice));
    cudaDeviceProp prop;
    CHECK(cudaGetDeviceProperties(&prop, 0));
    int failed = 0, total = 0;
    for (int tile = 64; tile <= 128; tile *= 2)
        for (int dim = tile; dim <= dim_max; dim += tile)
            for (int variant = 0; variant < 3; ++variant) {
                CHECK(cudaMemset(D, 0, size_t(dim) * dim * 2));
                const half one = __float2half(1.0f);
                int st;
                if (variant == 0) st = gemm_shmem_tc_async<half, half>(A, B, C, D, one, one, dim, dim, dim, tile, 64, 3, 2, 4, prop.multiProcessorCount);
                else if (variant == 1) st = gemm_shmem_tc_async_opt_port<half, half>(A, B, C, D, one, one, dim, dim, dim, tile, 64, 2, 3, 2, 8, prop.multiProcessorCount);
                else st = gemm_shmem_tc_async_opt_port<half, half>(A, B, C, D, one, one, dim, dim, dim, tile, 64, 1, 1, 16, 16, 1, 2, 2, 4, prop.multiProcessorCount);
                bool ok = st == B200_OK;
                if (ok) {
                    CHECK(cudaMemcpy(res.data(), D, size_t(dim) * dim * 2, cudaMemcpyDeviceToHost));
                    const float want = 10.0f * dim + 1.0f;
                    for (size_t e = 0; e < size_t(dim) * dim && ok; ++e) ok = __half2float(res[e]) == want;
                }
                ++total;
                if (!ok) { ++failed; printf("half output tile %d dim %d launcher %d: failed (status %d)\n", tile, dim, variant, st); }
            }
    int info[4];
    const int dev = b200_device_status(nullptr, info);
    printf("half output: %d launches, %d failed, device status %d\n", total, failed, dev);
    cudaFree(A); cudaFree(B); cudaFree(C); cudaFree(D);
    return failed == 0 && dev == B200_OK ? 0 : 1;
}

int main(int argc, char **argv) {
    const char *mode = argc > 1 ? argv[1] : "correctness";
    const int dim = argc > 2 ? atoi(argv[2]) : 1024;
    const bool quick = argc > 3;
    if (b200_num_sms() <= 0) { printf("no sm_100 device: %s\n", b200_status_string(B200_UNSUPPORTED_DEVICE)); return 2; }
    // ranges of the reference's own calls (port_2.cu:1518-1550), narrowed where `quick`
    Sweep s = {64, 128, 64, 256, 1, quick ? 1 : 2, 1, quick ? 2 : 3, 2, quick ? 2 : 4, 4, 8};
    if (!strcmp(mode, "correctness")) return run_correctness(dim, s, 2, 1.0f, 1.0f, 0.001f);
    if (!strcmp(mode, "half")) return run_half_output(dim < 192 ? dim : 192);   // 10 * 192 + 1 is exact in fp16
    if (!strcmp(mode, "accuracy")) { s.group_hi = 1; s.stages_lo = 2; s.stages_hi = 2; s.p_hi = 2; return run_accuracy(dim, s, 1.0f, 1.0f, 0.1f); }
    if (!strcmp(mode, "performance")) return run_performance(dim, 2);
    printf("unknown mode %s\n", mode);
    return 2;
}
