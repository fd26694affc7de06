// Arguments of the sm_100a GEMM kernel and its launch entry, shared by the kernel and the C ABI.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "plan.h"

namespace b200 {

struct alignas(64) GemmArgs {
    CUtensorMap map_a;  // A   as {K, M}  two-byte elements, box {64, a_box_rows}, 128-byte swizzle
    CUtensorMap map_b;  // B^T as {K, N}  two-byte elements, box {64, chunk_n / cta_group}
    CUtensorMap map_d;  // D   as {N, M}  fp32, box {32, 32}, 128-byte swizzle (TMA-store epilogue)
    const float *C;
    float *D;
    float *partial;     // split-K workspace: split_k slabs of M x N fp32; tail split: one partial per CTA and slice unit
    float alpha, beta;
    int M, N, K;
    int ld_cd;          // row pitch of C and D in elements (N unless D is a column block of a wider matrix)
    int tiles_m, tiles_n, num_tiles, num_units;
    int num_segs;       // K / seg_k
    int split_k;
    int tail_tiles, tail_slices;  // tail split (plan.h): the first tail_tiles tiles are cut into tail_slices K slices; 0 = off
    int tail_set;                 // which set of the fix-up flags this launch uses
    unsigned int tail_epoch;      // the value its flags carry (never 0)
    // plan
    int tile_m, tile_n, cta_rows_a, mma_m;
    int kblocks, stages, tile_group_m;
    int a_box_rows, a_boxes, a_priv, a_bars;
    int chunk_n, b_priv, b_res_chunks, b_bars;
    int producer_warps, epi_warps;
    int acc_cols, tmem_cols;
    int a_stage_bytes, stage_bytes;
    int off_epi, off_bars, off_tmem_ptr;
    int epi_mode;
    uint32_t idesc_chunk, idesc_res;
    long long wait_budget_cycles;
    long long *prof;    // optional cycle counters, 16 per CTA for the first prof_blocks CTAs
    int prof_blocks;
    int debug_flags;
    int l2_hint;
    int k_order;
    int cl_split;       // > 1: cluster size; the CTAs of a cluster take the K slices of one tile and reduce through
                        // distributed shared memory (split_k is 1 then: no workspace)
    int d_stream;       // 1: the TMA stores of D carry an evict_first L2 policy (D exceeds what the L2 would keep)
    int overlap_launch; // 1: set-up runs before griddepcontrol.wait (launched with programmatic stream serialisation)
    int epi_bufs;       // staging boxes per draining warp of the TMA-store drain (2 or 1)
    int atoms;          // MMA atoms per CTA and tile (1 or 2), mma_m rows of A each; their accumulators sit side by side in
                        // tensor memory (acc_cols = atoms * tile_n; two accumulator slots while 2 * acc_cols fits the 512 columns)
    int a_split;        // 1: a 128-row tile is two 64-row MMA atoms (the A side of the shift synchronisation): the upper
                        // atom's MMAs are issued when the row boxes of rows 0-63 have landed; accumulators of the two
                        // atoms sit side by side in tensor memory (acc_cols = 2 * tile_n)
    int out_half;       // 1: C and D hold fp16 (the reference's DT_ACC = half instances); accumulation stays fp32
    int swap_ab;        // 1: M/N above are those of the transposed problem and the tile is stored transposed (D[col][row])
    // split-K across GPUs with the reduce-scatter fused into the epilogue ("push" mode, world > 0):
    // the fp32 tile rows owned by GPU o are stored straight into o's slot area over NVLink
    // (plain peer stores), slot [source rank][rows per owner][N]; the last CTA to finish raises
    // this rank's flag on every owner.
    float *push_slot[8];
    int *push_flag[8];
    unsigned int *push_done;  // local counter of finished CTAs (zero between launches)
    int push_world, push_rank, push_rows, push_epoch;
};

// Launches the kernel for plan p on `stream`. Returns a cudaError_t as int.
int launch_gemm(const Plan &p, const GemmArgs &args, cudaStream_t stream);
int launch_splitk_reduce(const float *partial, const float *C, float *D, float alpha, float beta, int64_t mn,
                         int split_k, cudaStream_t stream);
// Reads and clears the device-side timeout record {code, block, barrier, phase}.
int read_device_status(int out[4], cudaStream_t stream);
// Owner side of push mode: waits (bounded) until every source rank's flag shows `epoch`, then
// D = alpha * sum over sources of slot[src] + beta * C for this GPU's rows.
int launch_push_reduce(const float *slots, const int *flags, int world, int epoch, const float *C, float *D, float alpha,
                       float beta, int64_t rows, int64_t n, long long budget_cycles, cudaStream_t stream);
// Stream-ordered flag write / bounded flag wait (flag >= epoch) for exchanges between the GPUs of a box.
int launch_flag_set(int *flag, int epoch, cudaStream_t stream);
int launch_flag_wait(const int *flag, int epoch, long long budget_cycles, int wait_id, cudaStream_t stream);
// Second step of split-K when the rows go to their owner GPUs instead of a local D.
int launch_splitk_reduce_push(const float *partial, int64_t m, int64_t n, int split_k, float *const *slots, int *const *flags,
                              unsigned int *done, int world, int rank, int epoch, cudaStream_t stream);
// Remembers the cudaError_t behind a B200_CUDA_ERROR return for b200_last_cuda_error(); returns B200_CUDA_ERROR.
int record_cuda_error(int cuda_error);
int prepare_kernels();  // opt-in shared memory size; once per device
int profile_slots();    // int64 slots per CTA of the profile buffer (16; 32 in a -DB200_TIMELINE build)

}  // namespace b200
