// b200_matmul.h - C++ launchers with the reference's own names and argument lists, forwarding
// to the C ABI (b200_gemm.h). A harness written against the reference launchers compiles against
// these unchanged, except that they return a status instead of void. DT_ACC = half (with DT = half)
// gives fp16 C and D; the accumulation is fp32 either way.
//
//   gemm_shmem_tc_async           15 arguments   matmul_shmem_tc_async.cu:494-510
//   gemm_shmem_tc_async_opt_port  16 arguments   matmul_shmem_tc_async_opt_port_0.cu:515-532
//                                 18 arguments   matmul_shmem_tc_async_opt_port_1.cu:889-908
//                                 20 arguments   matmul_shmem_tc_async_opt_port_2.cu:1088-1109
//
// DT is half or __nv_bfloat16 (device pointers), DT_ACC is float (or half with DT = half). A is m x k row-major, B is
// stored transposed (n x k), C and D are m x n. Launches go to the legacy default stream, as the
// reference's do.
//
// How the reference's tunables are honoured on sm_100a:
//   tile_dim            square CTA tile: tile_m = tile_n = tile_dim (64 or 128)
//   segment_dim_k       K extent per pipeline stage (multiple of 64)
//   num_stages          depth of the shared-memory ring
//   tile_group_m        tile rows per L2 rasterisation group
//   num_producer_warps  1: one warp issues the A and B^T copies; >= 2: one warp each
//   num_consumer_warps  4 or 8 warps draining the accumulator from tensor memory
//   bar_step_rows_a/b   rows of A / of B^T per sub-tile barrier; the tile extent switches the
//                       shift synchronisation off
//   bar_steps_a/b       leading sub-tiles with private barriers; the rest share a residual one
//   num_sms             size of the persistent grid
#ifndef B200_MATMUL_H
#define B200_MATMUL_H

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "b200_gemm.h"

namespace b200_matmul {

namespace detail {

template <typename DT>
struct InputType;
template <>
struct InputType<half> {
    static constexpr int value = B200_F16;
};
template <>
struct InputType<__nv_bfloat16> {
    static constexpr int value = B200_BF16;
};

// DT_ACC = half (the reference instantiates <half, half> beside <half, float>): fp16 C and D, scalars as half.
// The plain tile of these launchers never needs a workspace, so every reference configuration maps.
inline int launch(const half *A, const half *B, const half *C, half *D, half alpha, half beta, int M, int N, int K,
                  const b200_gemm_params &p) {
    if (M % p.tile_m || N % p.tile_n || K % p.segment_dim_k) return B200_INVALID_SHAPE;
    return b200_gemm_f16_out_f16(A, B, C, D, __half2float(alpha), __half2float(beta), M, N, K, &p, nullptr);
}

template <typename DT>
inline int launch(const DT *A, const DT *B, const float *C, float *D, float alpha, float beta, int M, int N, int K,
                  const b200_gemm_params &p) {
    // the reference's rule (async.cu:513-514, port_2.cu:1114-1115); the C ABI itself also takes ragged shapes
    if (M % p.tile_m || N % p.tile_n || K % p.segment_dim_k) return B200_INVALID_SHAPE;
    if (InputType<DT>::value == B200_BF16)
        return b200_gemm_bf16(A, B, C, D, alpha, beta, M, N, K, &p, nullptr, 0, nullptr);
    return b200_gemm_f16(A, B, C, D, alpha, beta, M, N, K, &p, nullptr, 0, nullptr);
}

inline b200_gemm_params base_params(int tile_dim, int segment_dim_k, int tile_group_m, int num_stages,
                                    int num_producer_warps, int num_consumer_warps, int num_sms) {
    b200_gemm_params p = {};
    p.tile_m = tile_dim;
    p.tile_n = tile_dim;
    p.segment_dim_k = segment_dim_k;
    p.bar_steps_a = 0;
    p.bar_steps_b = 0;
    p.bar_step_rows_a = tile_dim;
    p.bar_step_rows_b = tile_dim;
    p.tile_group_m = tile_group_m;
    p.num_stages = num_stages;
    p.num_producer_warps = num_producer_warps;
    p.num_consumer_warps = num_consumer_warps;
    p.num_sms = num_sms;
    p.cta_group = 1;
    p.split_k = 1;
    p.epilogue = 0;
    return p;
}

}  // namespace detail

// matmul_shmem_tc_async.cu:494-510 (row-major tile order = one tile row per group).
template <typename DT, typename DT_ACC>
int gemm_shmem_tc_async(const DT *A, const DT *B /* Transpose */, const DT_ACC *C, DT_ACC *D, DT_ACC alpha, DT_ACC beta,
                        int M, int N, int K, int tile_dim, int segment_dim_k, int num_stages, int num_producer_warps,
                        int num_consumer_warps, int num_sms) {
    static_assert(sizeof(DT_ACC) == 4 || (sizeof(DT_ACC) == 2 && sizeof(DT) == 2), "DT_ACC is float, or half with DT = half");
    if (tile_dim != 64 && tile_dim != 128) return B200_INVALID_CONFIG;  // async.cu:511
    const b200_gemm_params p =
        detail::base_params(tile_dim, segment_dim_k, 1, num_stages, num_producer_warps, num_consumer_warps, num_sms);
    return detail::launch(A, B, C, D, alpha, beta, M, N, K, p);
}

// matmul_shmem_tc_async_opt_port_0.cu:515-532.
template <typename DT, typename DT_ACC>
int gemm_shmem_tc_async_opt_port(const DT *A, const DT *B /* Transpose */, const DT_ACC *C, DT_ACC *D, DT_ACC alpha,
                                 DT_ACC beta, int M, int N, int K, int tile_dim, int segment_dim_k, int tile_group_m,
                                 int num_stages, int num_producer_warps, int num_consumer_warps, int num_sms) {
    static_assert(sizeof(DT_ACC) == 4 || (sizeof(DT_ACC) == 2 && sizeof(DT) == 2), "DT_ACC is float, or half with DT = half");
    if (tile_dim != 64 && tile_dim != 128) return B200_INVALID_CONFIG;
    const b200_gemm_params p = detail::base_params(tile_dim, segment_dim_k, tile_group_m, num_stages, num_producer_warps,
                                                   num_consumer_warps, num_sms);
    return detail::launch(A, B, C, D, alpha, beta, M, N, K, p);
}

// matmul_shmem_tc_async_opt_port_2.cu:1088-1109.
template <typename DT, typename DT_ACC>
int gemm_shmem_tc_async_opt_port(const DT *A, const DT *B /* Transpose */, const DT_ACC *C, DT_ACC *D, DT_ACC alpha,
                                 DT_ACC beta, int M, int N, int K, int tile_dim, int segment_dim_k, int bar_steps_a,
                                 int bar_steps_b, int bar_step_rows_a, int bar_step_rows_b, int tile_group_m,
                                 int num_stages, int num_producer_warps, int num_consumer_warps, int num_sms) {
    static_assert(sizeof(DT_ACC) == 4 || (sizeof(DT_ACC) == 2 && sizeof(DT) == 2), "DT_ACC is float, or half with DT = half");
    if (tile_dim != 64 && tile_dim != 128) return B200_INVALID_CONFIG;
    // port_1.cu:919 and port_2.cu:1122: the shift-synchronised generations need >= 2 producer warps
    if (num_producer_warps != 2 && num_producer_warps != 4 && num_producer_warps != 8) return B200_INVALID_CONFIG;
    b200_gemm_params p = detail::base_params(tile_dim, segment_dim_k, tile_group_m, num_stages, num_producer_warps,
                                             num_consumer_warps, num_sms);
    p.bar_steps_a = bar_steps_a;
    p.bar_steps_b = bar_steps_b;
    p.bar_step_rows_a = bar_step_rows_a;
    p.bar_step_rows_b = bar_step_rows_b;
    return detail::launch(A, B, C, D, alpha, beta, M, N, K, p);
}

// matmul_shmem_tc_async_opt_port_1.cu:889-908: every sub-tile has a private barrier.
template <typename DT, typename DT_ACC>
int gemm_shmem_tc_async_opt_port(const DT *A, const DT *B /* Transpose */, const DT_ACC *C, DT_ACC *D, DT_ACC alpha,
                                 DT_ACC beta, int M, int N, int K, int tile_dim, int segment_dim_k, int bar_step_rows_a,
                                 int bar_step_rows_b, int tile_group_m, int num_stages, int num_producer_warps,
                                 int num_consumer_warps, int num_sms) {
    const int steps_a = (bar_step_rows_a > 0 && bar_step_rows_a < tile_dim) ? tile_dim / bar_step_rows_a : 0;
    const int steps_b = (bar_step_rows_b > 0 && bar_step_rows_b < tile_dim) ? tile_dim / bar_step_rows_b : 0;
    return gemm_shmem_tc_async_opt_port<DT, DT_ACC>(A, B, C, D, alpha, beta, M, N, K, tile_dim, segment_dim_k, steps_a,
                                                    steps_b, bar_step_rows_a, bar_step_rows_b, tile_group_m, num_stages,
                                                    num_producer_warps, num_consumer_warps, num_sms);
}

// Counterparts of the reference's host helpers.
// get_shmem_req (port_2.cu:1057-1086): dynamic shared memory of the configuration, or -1.
inline int get_shmem_req(int tile_dim, int segment_dim_k, int bar_steps_a, int bar_steps_b, int bar_step_rows_a,
                         int bar_step_rows_b, int num_stages, int num_consumer_warps) {
    b200_gemm_params p = detail::base_params(tile_dim, segment_dim_k, 1, num_stages, 2, num_consumer_warps, 0);
    p.bar_steps_a = bar_steps_a;
    p.bar_steps_b = bar_steps_b;
    p.bar_step_rows_a = bar_step_rows_a;
    p.bar_step_rows_b = bar_step_rows_b;
    return static_cast<int>(b200_gemm_smem_bytes(B200_F16, &p));
}
// get_num_acc / get_warp_tile_rows (port_2.cu:158-169) describe the reference's warp tile; the
// sweeps use them to derive the barrier granularities, so they are kept with the same values.
inline int get_num_acc(int tile_dim, int num_consumer_warps) {
    const int w = 4 >> (tile_dim == 64);
    return w * (w >> (num_consumer_warps == 8));
}
inline int get_warp_tile_rows(int tile_dim, int num_consumer_warps) {
    const int num_acc = get_num_acc(tile_dim, num_consumer_warps);
    return num_acc < 8 ? num_acc / 2 : num_acc / 4;
}

}  // namespace b200_matmul

#endif  // B200_MATMUL_H
