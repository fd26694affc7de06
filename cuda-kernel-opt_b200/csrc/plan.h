// Host-side planning: turns the caller's tunables into the launch plan of the sm_100a kernel
// (tile split, TMA boxes, barrier counts, shared-memory map, TMEM columns, block size) or a
// status. Pure C++: usable and testable without a GPU.
//
// It is the counterpart of the reference launcher's asserts and of get_shmem_req /
// get_num_acc / get_warp_tile_rows (matmul_shmem_tc_async_opt_port_2.cu:1112-1125, :1057-1086,
// :158-169): same tunables, same refusal of what does not fit, but as return codes.
#pragma once

#include <cstdint>
#include "../../include/b200_gemm.h"

namespace b200 {

constexpr int kSmemLimit = 232448;      // 227 KiB: largest opt-in dynamic shared memory per CTA
constexpr int kTmemColumns = 512;       // 32-bit columns of tensor memory per SM
constexpr int kSwizzleBytes = 128;      // one TMA box / UMMA atom row: 64 two-byte elements
constexpr int kBoxK = 64;               // K elements per TMA box
constexpr int kMaxSubBars = 17;         // private sub-tile barriers (<= 16) + one residual
constexpr int kMaxStages = 16;          // NUM_STAGES_MAX of the reference (matmul_shmem_tc_async.cu:43)
constexpr int kEpiBoxCols = 32;         // columns drained per tcgen05.ld / per TMA-store box
constexpr int kMinSmemRequest = 120000; // more than half an SM's shared memory: one CTA per SM,
                                        // so two CTAs never contend for the 512 TMEM columns

struct Plan {
    int status = B200_INVALID_CONFIG;
    // tile
    int tile_m = 0, tile_n = 0, cta_group = 1;
    int cta_rows_a = 0;   // rows of A each CTA stages (tile_m / cta_group)
    int cta_rows_b = 0;   // rows of B^T each CTA stages (tile_n / cta_group)
    int mma_m = 0;        // M of one tcgen05.mma as seen by one CTA's tensor memory (64 or 128)
    int seg_k = 0, kblocks = 0, stages = 0;
    // sub-tile ("shift synchronisation") split of a stage
    int a_box_rows = 0, a_boxes = 0;      // A rows per TMA box, boxes per k-block per CTA
    int a_priv = 0, a_bars = 0;           // leading A boxes with private barriers; total A barriers
    int chunk_n = 0;                      // tile columns per B^T sub-tile
    int b_priv = 0, b_res_chunks = 0;     // private sub-tiles; sub-tiles on the residual barrier
    int b_bars = 0;
    // roles
    int producer_warps = 0, epi_warps = 0, threads = 0;
    // resources
    int tmem_cols = 0, acc_cols = 0;      // allocation; columns per accumulator slot (2 slots)
    int stage_bytes = 0, a_stage_bytes = 0, b_stage_bytes = 0;
    int epi_mode = 0, epi_bytes = 0;
    int epi_bufs = 2;                     // 32x32 fp32 staging boxes per draining warp of the TMA-store drain: 2, or 1 when 2 do not fit
    int num_barriers = 0;
    int off_epi = 0, off_bars = 0, off_tmem_ptr = 0;
    int smem_bytes = 0;                   // dynamic shared memory requested (includes alignment slack)
    int split_k = 1;
    int tile_group_m = 1;
    int grid = 0;
    int swap = 0;                         // 1: the kernel computes D^T = B^T * A^T (tile_m spans N, tile_n spans M)
    int cluster_reduce = 0;               // 1: the split_k slices of a tile run in one thread-block cluster and meet
                                          //    in distributed shared memory (no workspace, no second kernel)
    int a_split = 0;                      // 1: a 128-row tile is issued as two 64-row MMA atoms so that the upper rows'
                                          //    MMAs start before the lower rows of A have landed (A-side shift)
    int atoms = 1, atom_rows = 0;         // MMA atoms a CTA's rows of A are issued as (1 or 2) and the rows of one
    int acc_slots = 2;                    // accumulator slots in tensor memory: 2 (the drain of a tile overlaps the MMAs of
                                          //    the next), or 1 when one tile's accumulator fills the 512 columns
};

// Tail split (tail_split = 1): the tiles that do not fill a wave of the persistent grid are cut along K.
// T tiles on S slots (CTAs, or CTA pairs) leave r = T mod S tiles for a last, partly idle wave that still
// costs a whole tile time. Instead those r tiles are cut into s equal K slices each; the r * s slice units
// are dealt to the slots slice-major (all first slices, then all second slices, ...) and run FIRST, before
// the whole tiles; with s = floor(S / r) they fit one round, so the tail costs 1 / s of a tile time instead
// of 1. The slice-major order keeps the slots in step along K: the CTAs
// that run at the same time read the same K range of neighbouring tiles, so operand panels are shared in
// L2 as in a wave of whole tiles. (A plain stream-K cut - one contiguous range of K iterations per slot -
// balances better on paper but puts every slot at a different K offset: nothing is shared, the phase turns
// DRAM-bound and the gain is lost; measured.) The slot that runs a tile's last slice finishes the tile: the
// other slices store their raw fp32 accumulators in the workspace and raise a flag, the finisher adds them
// in ascending K order before the usual alpha / beta / store. Running the tail first hides that fix-up
// behind the whole tiles that follow. tiles == 0 means "off / nothing to gain".
struct TailPlan {
    int tiles = 0;           // r: the first r tiles in tile order are cut
    int slices = 1;          // s: K slices per cut tile
    int64_t slot_bytes = 0;  // one partial per CTA and slice unit: 128 lanes x ceil(tile_n / 32) chunks of 32 columns, fp32
    int64_t slots = 0;       // partials in CTA units: r * (s - 1) * cta_group
};

constexpr int kTailMaxSlices = 8;
constexpr int kTailMaxSlots = 1040;   // flags per set the library keeps: covers 148 one-CTA tiles x 7 slices

inline TailPlan make_tail_plan(int enabled, int64_t tiles, int slots, int64_t num_segs, int split_k, int tile_n, int cta_group) {
    TailPlan t;
    if (!enabled || split_k > 1 || slots < 2 || tiles <= 0) return t;
    const int64_t r = tiles % slots;
    if (r == 0) return t;
    // One round only: s = floor(S / r) slices (at most 8, and slices of at least four K segments), so every slot runs
    // at most one slice unit and the tail costs 1 / s of a tile time. Plans with several rounds balance better on
    // paper (54 tiles left on 74 pairs: quarters in three rounds, 0.75) but measured slower than the plain schedule:
    // every extra slice is a 128 x tile_n fp32 partial written and read back, and under the power limit the time of
    // a launch follows the energy it spends more than the SM time it leaves idle.
    int best_s = static_cast<int>(slots / r);
    if (best_s > kTailMaxSlices) best_s = kTailMaxSlices;
    while (best_s > 1 && num_segs / best_s < 4) --best_s;
    while (best_s > 1 && r * (best_s - 1) * cta_group > kTailMaxSlots) --best_s;
    const int64_t waves = (tiles + slots - 1) / slots;
    if (best_s < 2 || (1.0 - 1.0 / best_s) / double(waves) < 0.02) return t;   // under 2 % of the launch: not worth the traffic
    t.tiles = static_cast<int>(r);
    t.slices = best_s;
    t.slot_bytes = int64_t((tile_n + 31) / 32) * 4 * 32 * 32 * 4;
    t.slots = r * (best_s - 1) * cta_group;
    return t;
}

inline int round_up(int x, int m) { return (x + m - 1) / m * m; }

inline int pow2_at_least(int x) {
    int p = 32;
    while (p < x) p <<= 1;
    return p;
}

// Validates tunables that do not depend on the problem shape and lays out shared memory.
inline Plan make_plan(const b200_gemm_params &user, int num_sms_device) {
    Plan p;
    p.status = B200_INVALID_CONFIG;
    b200_gemm_params q = user;
    if (user.swap_ab != 0 && user.swap_ab != 1) return p;
    if (user.swap_ab) {
        // Swapped operand roles: plan the transposed problem. The caller's tile_n (columns of D, rows of
        // B^T) becomes the 64/128-row side of the MMA, tile_m its N side; sub-tile barriers follow
        // their operands; the drain is plain stores (a transposed tile has no row-major TMA box).
        if (user.tail_split) return p;
        if (user.epilogue != 0 && user.epilogue != 1) return p;
        q.tile_m = user.tile_n;
        q.tile_n = user.tile_m;
        q.bar_steps_a = user.bar_steps_b;
        q.bar_steps_b = user.bar_steps_a;
        q.bar_step_rows_a = user.bar_step_rows_b;
        q.bar_step_rows_b = user.bar_step_rows_a;
        q.epilogue = 0;
        p.swap = 1;
    }
    const int cg = q.cta_group == 0 ? 1 : q.cta_group;
    if (cg != 1 && cg != 2) return p;
    p.cta_group = cg;
    // tile_m: 128 or 64 for one CTA; 256 for a pair (each CTA holds 128 rows); 512 for a "tall" pair: each CTA
    // holds 256 rows of A, issued as two 128-row atoms against the same B^T stage, so a byte of B^T feeds twice the
    // MMA work (operand bytes per flop drop by a quarter against the 256-row pair).
    if (cg == 1 && q.tile_m != 128 && q.tile_m != 64) return p;
    if (cg == 2 && q.tile_m != 256 && q.tile_m != 512) return p;
    p.tile_m = q.tile_m;
    p.cta_rows_a = q.tile_m / cg;
    p.mma_m = p.cta_rows_a > 128 ? 128 : p.cta_rows_a;
    p.atoms = p.cta_rows_a / p.mma_m;
    p.atom_rows = p.mma_m;
    if (p.atoms == 2 && (p.swap || user.cluster_reduce)) return p;
    // tile_n: N of the MMA. M=128 per CTA needs N % 16 == 0, M=64 needs N % 8; a pair splits N.
    const int n_gran = 16 * cg;
    if (q.tile_n < n_gran || q.tile_n > 256 || q.tile_n % n_gran) return p;
    p.tile_n = q.tile_n;
    p.cta_rows_b = q.tile_n / cg;
    if (q.segment_dim_k < kBoxK || q.segment_dim_k % kBoxK) return p;  // port_2.cu:1113
    p.seg_k = q.segment_dim_k;
    p.kblocks = q.segment_dim_k / kBoxK;
    if (q.num_stages < 1 || q.num_stages > kMaxStages) return p;       // port_2.cu:1121
    p.stages = q.num_stages;
    if (q.tile_group_m < 1) return p;                                  // port_2.cu comment :631
    p.tile_group_m = q.tile_group_m;
    if (q.num_producer_warps != 1 && q.num_producer_warps != 2 && q.num_producer_warps != 4 &&
        q.num_producer_warps != 8)
        return p;                                                      // async.cu:516
    // Only the first two producer warps issue copies, the others would idle: at most three are launched, which
    // keeps the block at 12 warps (384 threads) and the kernel's register budget at 168 per thread.
    p.producer_warps = q.num_producer_warps > 3 ? 3 : q.num_producer_warps;
    if (q.num_consumer_warps != 4 && q.num_consumer_warps != 8) return p;  // async.cu:517
    p.epi_warps = q.num_consumer_warps;
    p.threads = (p.producer_warps + 1 + p.epi_warps) * 32;
    if (q.split_k < 0 || q.split_k > 64) return p;
    p.split_k = q.split_k == 0 ? 1 : q.split_k;
    if (q.epilogue != 0 && q.epilogue != 1) return p;
    if (q.l2_hint < 0 || q.l2_hint > 3) return p;
    if (q.k_order != 0 && q.k_order != 1) return p;
    if (q.overlap_launch != 0 && q.overlap_launch != 1) return p;
    p.epi_mode = q.epilogue;
    if (user.cluster_reduce != 0 && user.cluster_reduce != 1) return p;
    if (user.cluster_reduce) {
        // K slices as the CTAs of a cluster: portable cluster sizes, a transposed accumulator of at
        // most 128 columns (64 KiB of fp32 per CTA) staged in shared memory for the peers to read.
        if (!p.swap || (p.split_k != 2 && p.split_k != 4 && p.split_k != 8) || q.tile_n > 128) return p;
        if (cg * p.split_k > 8) return p;   // pairs x slices must fit a portable cluster
        p.cluster_reduce = 1;
    }

    // Sub-tile split of the A stage buffer (rows per barrier step). 0 or the full extent = off.
    int step_a = q.bar_step_rows_a;
    if (step_a <= 0 || step_a >= p.tile_m) step_a = p.tile_m;
    if (step_a == p.tile_m) {
        p.a_box_rows = p.cta_rows_a;
        p.a_boxes = 1;
        p.a_priv = 0;
        p.a_bars = 1;
    } else {
        if (step_a % 16 || p.cta_rows_a % step_a) return p;
        p.a_box_rows = step_a;
        p.a_boxes = p.cta_rows_a / step_a;
        if (q.bar_steps_a < 0 || q.bar_steps_a > p.a_boxes) return p;  // port_2.cu:1116-1120
        p.a_priv = q.bar_steps_a;
        p.a_bars = p.a_priv + (p.a_priv < p.a_boxes ? 1 : 0);
    }
    // Sub-tile split of the B^T stage buffer (tile columns per barrier step).
    int step_b = q.bar_step_rows_b;
    if (step_b <= 0 || step_b >= p.tile_n) step_b = p.tile_n;
    if (step_b == p.tile_n) {
        p.chunk_n = p.tile_n;
        p.b_priv = 0;
        p.b_res_chunks = 1;
        p.b_bars = 1;
    } else {
        if (step_b % n_gran || p.tile_n % step_b) return p;
        const int chunks = p.tile_n / step_b;
        if (chunks > 16) return p;
        p.chunk_n = step_b;
        if (q.bar_steps_b < 0 || q.bar_steps_b > chunks) return p;
        p.b_priv = q.bar_steps_b;
        p.b_res_chunks = chunks - p.b_priv;
        p.b_bars = p.b_priv + (p.b_res_chunks > 0 ? 1 : 0);
    }
    if (p.a_bars > kMaxSubBars || p.b_bars > kMaxSubBars) return p;

    // A-side shift synchronisation that starts MMAs early (the reference's per-fragment-row waits, port_1.cu:406-433):
    // a one-CTA 128-row tile whose A buffer is released in steps of at most 64 rows is issued as two 64-row atoms; the
    // upper atom waits only for the barriers of rows 0-63. Its accumulators sit side by side in tensor memory, so the
    // tile may be at most 128 columns wide (2 atoms x 2 slots x 128 = 512 columns); wider tiles, pairs, swapped roles
    // and K slices keep the one-atom form, where the A steps change the copy granularity only.
    if (cg == 1 && p.tile_m == 128 && !p.swap && p.a_boxes > 1 && p.a_box_rows <= 64 && 64 % p.a_box_rows == 0 &&
        p.tile_n <= 128 && p.split_k == 1) {
        p.a_split = 1;
        p.mma_m = 64;
        p.atoms = 2;
        p.atom_rows = 64;
    }
    // the tall pair: whole-stage barriers (it runs in the lean producer / MMA loops only), whole tiles
    if (p.atoms == 2 && !p.a_split && (p.a_boxes > 1 || p.b_bars > 1 || p.b_priv != 0 || p.b_res_chunks != 1 || p.split_k > 1)) return p;

    // Tensor memory: two accumulator slots so the drain of tile i overlaps the MMAs of tile i+1.
    // M=64 per CTA keeps the 16-lanes-per-quarter layout of one 64-row atom.
    p.acc_cols = p.atoms * p.tile_n;
    p.acc_slots = (2 * p.acc_cols <= kTmemColumns) ? 2 : 1;
    p.tmem_cols = pow2_at_least(p.acc_slots * p.acc_cols);
    if (p.tmem_cols > kTmemColumns) return p;

    // Shared memory map (offsets from a 1024-byte aligned base).
    p.a_stage_bytes = p.cta_rows_a * p.seg_k * 2;
    p.b_stage_bytes = p.cta_rows_b * p.seg_k * 2;
    p.stage_bytes = p.a_stage_bytes + p.b_stage_bytes;
    if (p.a_stage_bytes % 1024 || p.b_stage_bytes % 1024) return p;
    // every sub-tile base must stay 1024-byte aligned (8 rows of 128 bytes)
    if ((p.a_box_rows % 8) || ((p.chunk_n / cg) % 8)) return p;
    p.off_epi = p.stages * p.stage_bytes;
    p.num_barriers = p.stages * 2 * (p.a_bars + p.b_bars) /* full + empty */ + 4 /* tmem full/empty x2 */ +
                     2 /* partial tile full / empty (cluster reduce) */;
    // The TMA-store drain stages two 32x32 fp32 boxes per warp (one being read by the copy engine while the next is
    // written); where two do not fit beside the ring (eight draining warps next to four 48 KB stages of the tall pair)
    // one does: the read of a box has long finished when the warp comes round to it again.
    for (p.epi_bufs = 2; p.epi_bufs >= 1; --p.epi_bufs) {
        p.epi_bytes = p.epi_mode ? p.epi_warps * p.epi_bufs * 32 * kEpiBoxCols * 4 : 0;
        if (p.cluster_reduce) p.epi_bytes = p.tile_n * 128 * 4;                 // this CTA's partial tile, [column][row]
        p.off_bars = p.off_epi + p.epi_bytes;
        p.off_tmem_ptr = p.off_bars + p.num_barriers * 8;
        p.smem_bytes = p.off_tmem_ptr + 16 + 1024;  // slack to align the dynamic base to 1024 bytes
        if (p.smem_bytes <= kSmemLimit || !p.epi_mode || p.cluster_reduce) break;
    }
    if (p.epi_bufs < 1) p.epi_bufs = 1;
    if (p.smem_bytes > kSmemLimit) return p;  // the harness's filter, port_2.cu:1229-1231
    if (p.smem_bytes < kMinSmemRequest) p.smem_bytes = kMinSmemRequest;

    int sms = q.num_sms > 0 ? q.num_sms : num_sms_device;
    if (sms < cg) return p;
    p.grid = sms - sms % cg;
    p.status = B200_OK;
    return p;
}

// Shape checks of the reference launcher (port_2.cu:1114-1115) plus what the new tiling adds.
inline int check_shape(const Plan &p, int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return B200_INVALID_SHAPE;
    // N must tile exactly; a ragged last tile row of M is handled by TMA zero fill on load and
    // clipped stores (the reference requires both to be tile multiples, port_2.cu:1114).
    // Ragged N and K are handled the same way (the reference also requires N % tile and
    // K % segment_dim_k == 0, port_2.cu:1114-1115; its launcher-shaped wrappers keep that rule).
    // What remains: 16-byte aligned rows, i.e. N % 4 == 0 for fp32 D and K % 8 == 0 for the
    // two-byte operands (TMA global strides are multiples of 16 bytes).
    if (N % 4 || K % 8) return B200_INVALID_SHAPE;
    if (M > (int64_t(1) << 30) || N > (int64_t(1) << 30) || K > (int64_t(1) << 30)) return B200_INVALID_SHAPE;
    if (p.split_k > 1 && ((K + p.seg_k - 1) / p.seg_k) < p.split_k) return B200_INVALID_SHAPE;
    return B200_OK;
}

}  // namespace b200
