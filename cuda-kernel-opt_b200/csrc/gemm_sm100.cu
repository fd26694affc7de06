// D = alpha * A * B^T + beta * C on the 5th-generation tensor cores of sm_100a.
//
// One persistent, warp-specialised kernel replaces the reference's four
// gemm_shmem_tc_async*_kernel generations (matmul_shmem_tc_async.cu:211-341,
// matmul_shmem_tc_async_opt_port_{0,1,2}.cu:225-354, :515-699, :638-878):
//
//   producer warp(s)  one elected lane issues TMA tile loads of A and B^T K-segments into a
//                     num_stages deep shared-memory ring (replaces load_tile_async / load_tile);
//   MMA warp          one thread issues tcgen05.mma from shared-memory descriptors, accumulating
//                     in tensor memory (replaces the wmma fragment loops of consume);
//   epilogue warps    drain tensor memory to registers, apply alpha / beta*C, write D either with
//                     128-bit stores or through swizzled shared memory and TMA stores (replaces
//                     store_matrix_sync + store_tile).
//
// Synchronisation is mbarriers only. A stage owns "full" barriers completed by TMA byte counts
// and "empty" barriers completed by tcgen05.commit. The reference's shift synchronisation
// (port_1.cu:164-328, port_2.cu:173-405: private barriers for the leading rows / columns of the
// stage buffers, one residual barrier for the rest) becomes sub-tile barriers inside a stage:
// the B^T buffer is split into column sub-tiles, each with its own TMA boxes, full barrier and
// MMA, issued in load order, so the first sub-tile's MMA starts before the rest of the stage has
// landed; the A buffer is split into row boxes with their own barriers, and a one-CTA 128-row tile
// released in steps of at most 64 rows is issued as two 64-row MMA atoms, the upper one as soon as
// the barriers of rows 0-63 are complete (the reference's per-fragment-row start, port_1.cu:406-433).
//
// Two accumulator slots in tensor memory let the drain of tile i overlap the MMAs of tile i+1,
// where the reference drains the whole pipeline at every tile (async.cu:339). The tall pair tile
// (512 x 256 per CTA pair: each CTA's 256 rows of A are two 128-row MMA atoms against one B^T stage)
// trades that for a quarter fewer operand bytes per flop: its two accumulators fill the tensor
// memory, one slot, and the drain (eight warps) is exposed.
//
// The schedule (schedule.h) is the reference's persistent tile loop (async.cu:251-252) plus a tail
// split: the tiles that would leave a last wave partly empty are cut into K slices that run first,
// one per CTA (pair); the CTA of a tile's last slice adds the other slices' partials from the
// workspace (flags, bounded waits) before the usual drain, so no second kernel is needed.
//
// Skinny (decode) shapes: with swapped roles the kernel computes D^T = B^T * A^T, so B^T fills the
// 128-row side of the MMA and the few rows of A its N side; the epilogue then writes the
// accumulator transposed. When a shape has few tiles, the K slices of one tile run as the CTAs
// (or CTA pairs) of a thread-block cluster and are summed through distributed shared memory in
// the epilogue (no workspace, no second kernel).
//
// Every wait is bounded: when its budget runs out the CTA records {code, block, barrier, phase}
// in a device status word, raises a block-wide abort flag so all roles leave their loops, frees
// its tensor memory and returns normally.
#include <cuda_fp16.h>

#include <mutex>
#include <vector>

#include "gemm_sm100.cuh"
#include "ptx_sm100.cuh"
#include "schedule.h"

namespace b200 {

__device__ int g_device_status[4];

namespace {

#ifdef B200_TIMELINE
// Diagnostic build: slots 16 .. 31 hold %globaltimer stamps of set-up and role milestones.
constexpr int kProfSlots = 34;
constexpr int kEarlySlot = 32;
#define B200_TL(slot) do { if (PROF && prof) prof[slot] = static_cast<long long>(global_timer_ns()); } while (0)
#else
constexpr int kProfSlots = 18;
constexpr int kEarlySlot = 16;   // [kEarlySlot] stages whose first MMAs were issued before the last rows of A had landed, [+1] stages
#define B200_TL(slot) do { } while (0)
#endif
constexpr int kMaxThreads = 384;  // (3 producer + 1 MMA + 8 epilogue warps) * 32: up to 168 registers per thread

// Flags of the tail split's fix-up: [set][partial slot][epilogue warp] holds the epoch of the launch whose
// partial that warp has stored. A set belongs to one launch at a time (the host deals them out in turn);
// the finishing warp puts the flag back to zero. Zero at load.
constexpr int kTailSets = 16;
__device__ unsigned int g_tail_flags[kTailSets][kTailMaxSlots][8];

// A bounded wait ran out: raise the block-wide abort flag and leave {code, block, wait id, detail} in
// the device status record (the first timeout of a launch wins).
__device__ __noinline__ void record_timeout(volatile int *abort_flag, int wait_id, int detail) {
    *abort_flag = 1;
    if (atomicCAS(&g_device_status[0], 0, B200_DEVICE_TIMEOUT) == 0) {
        g_device_status[1] = static_cast<int>(blockIdx.x);
        g_device_status[2] = wait_id;
        g_device_status[3] = detail;
    }
    __threadfence();
}

// Bounded mbarrier wait. Returns false when the budget ran out here or elsewhere in the block.
template <bool CLUSTER_ACQUIRE = false>
__device__ __noinline__ bool wait_slow(uint32_t bar, uint32_t parity, long long budget, volatile int *abort_flag,
                                       int bar_id) {
    const long long t0 = clock64();
    uint32_t spins = 0;
    for (;;) {
        if (CLUSTER_ACQUIRE ? mbar_try_wait_acquire_cluster(bar, parity) : mbar_try_wait(bar, parity)) return true;
#ifdef B200_WAIT_SLEEP
        __nanosleep(B200_WAIT_SLEEP);
#endif
        if ((++spins & 31u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > budget) {
                record_timeout(abort_flag, bar_id, static_cast<int>(parity));
                return false;
            }
        }
    }
}

// Every lane of a converged warp waits; the result is the same in every lane. All lanes execute the same
// try_wait on the same barrier, so the warp never diverges here and the .sync.aligned tensor-memory
// instructions that follow a wait find it converged. (Letting one elected lane poll while the others park at
// the vote was tried to save issue slots: it measured 1.3 % slower on 8192^3, the extra branch and vote sit on
// the MMA thread's critical path, with no difference in joules per TFLOP, so it was dropped.)
template <bool CLUSTER_ACQUIRE = false>
__device__ __forceinline__ bool wait_all(uint32_t bar, uint32_t parity, long long budget, volatile int *abort_flag,
                                         int bar_id) {
    bool ok = CLUSTER_ACQUIRE ? mbar_try_wait_acquire_cluster(bar, parity) : mbar_try_wait(bar, parity);
    if (__all_sync(0xffffffffu, ok)) return true;
    if (!ok) ok = wait_slow<CLUSTER_ACQUIRE>(bar, parity, budget, abort_flag, bar_id);
    return __all_sync(0xffffffffu, ok);
}

// Tail split, the CTA that runs a cut tile's last K slice: a bounded wait until warp e of every CTA that ran
// one of the tile's earlier slices has stored its partial (flag == this launch's epoch; lane 0 puts the flag
// back to zero). slot0 is the CTA-unit slot of slice 0, the slots of the following slices are
// slot_step apart. All lanes call it; false when the wait ran out or the block is aborting.
__device__ __forceinline__ bool tail_wait_peers(volatile unsigned int *flags, unsigned int epoch, int slot0, int slot_step,
                                                int peers, int e, long long budget, volatile int *abort_flag) {
    // Every lane reads the same flag word and the loop exits on votes, so the warp stays converged for the
    // .sync.aligned tensor-memory loads that follow.
    const long long t0 = clock64();
    for (int i = 0; i < peers; ++i) {
        volatile unsigned int *flag = flags + (slot0 + i * slot_step) * 8 + e;
        for (;;) {
            const bool there = (*flag == epoch);
            if (__all_sync(0xffffffffu, there)) break;
            __nanosleep(100);
            const bool aborting = (*abort_flag != 0);
            const bool late = clock64() - t0 > budget;
            if (__any_sync(0xffffffffu, aborting || late)) {
                if (lane_id() == 0 && !aborting) record_timeout(abort_flag, 800 + e, slot0 + i * slot_step);
                __syncwarp();
                return false;
            }
        }
        __syncwarp();
        if (lane_id() == 0) *flag = 0u;               // ready for the next launch that is dealt this flag set
    }
    __threadfence();
    return true;
}

template <int CG>
__device__ __forceinline__ void commit_to(uint32_t bar, uint16_t pair_mask) {
    if constexpr (CG == 1) {
        umma_commit<1>(bar);
    } else {
        // Both CTAs of the pair hold a barrier at this offset; complete the two of them
        // (pair_mask: the pair's two ranks in the cluster).
        asm volatile(
            "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
            "h"(pair_mask)
            : "memory");
    }
}

}  // namespace

// CG: CTAs per tcgen05 group. SIMPLE: one full and one empty barrier per stage (no sub-tiles),
// which allows the lean producer and MMA loops below. PROF: per-role cycle counters.
template <int CG, bool SIMPLE, bool PROF>
__global__ void __launch_bounds__(kMaxThreads, 1) gemm_sm100_kernel(const __grid_constant__ GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    Cfg c;
    c.num_units = g.num_units; c.num_tiles = g.num_tiles; c.tiles_m = g.tiles_m; c.tiles_n = g.tiles_n;
    c.tile_group_m = g.tile_group_m; c.tile_m = g.tile_m; c.tile_n = g.tile_n; c.num_segs = g.num_segs;
    c.split_k = g.split_k; c.tail_tiles = g.tail_tiles; c.tail_slices = g.tail_slices; c.kblocks = g.kblocks; c.stages = g.stages; c.stage_bytes = g.stage_bytes;
    c.a_stage_bytes = g.a_stage_bytes; c.cta_rows_a = g.cta_rows_a; c.a_box_rows = g.a_box_rows;
    c.a_boxes = g.a_boxes; c.a_priv = g.a_priv; c.a_bars = g.a_bars; c.chunk_n = g.chunk_n; c.b_priv = g.b_priv;
    c.b_res_chunks = g.b_res_chunks; c.b_bars = g.b_bars; c.acc_cols = g.acc_cols; c.mma_m = g.mma_m;
    c.epi_mode = g.epi_mode; c.epi_warps = g.epi_warps; c.M = g.M; c.N = g.N;
    c.idesc_chunk = g.idesc_chunk; c.idesc_res = g.idesc_res; c.budget = g.wait_budget_cycles;
    c.cl_split = g.cl_split > 1 ? g.cl_split : 1;
    c.cl_rank = 0;
    const int off_bars = g.off_bars, off_tmem_ptr = g.off_tmem_ptr, off_epi = g.off_epi;
    const int tmem_cols = g.tmem_cols;
    const int P = g.producer_warps;
    const int push_world = g.push_world, push_rank = g.push_rank, push_rows = g.push_rows;
    const int ld_cd = g.ld_cd;
    const bool swap_ab = g.swap_ab != 0;
    // 2 atoms: a CTA's rows of a tile are two MMA atoms with accumulators side by side: two 64-row atoms issued as
    // their rows of A land (a_split), or two 128-row atoms of a 256-row CTA share (the tall pair)
    // (read from the parameter inside each role: the values are not kept live across the others)
    const bool out_half = g.out_half != 0;   // C and D are fp16 (never with a workspace, tail or push path)
    // bit 0: issue no MMA, bit 1: issue no TMA load (pipeline ceilings; results are garbage); bits 2 and 3: the
    // epilogue withholds its "slice staged" / "slice read" arrivals of the cluster reduce, so that those
    // bounded waits run out and the launch ends with a DEVICE_TIMEOUT record (tests of the failure path); bit 4:
    // the same for the "partial stored" flags of the tail split
    const int dbg = g.debug_flags;
    const float g_alpha = g.alpha, g_beta = g.beta;
    volatile unsigned int *const tail_flags = &g_tail_flags[g.tail_set % kTailSets][0][0];
    const unsigned int tail_epoch = g.tail_epoch;
    const float *const gC = g.C;
    float *const gD = g.D;
    float *const g_partial = g.partial;
    long long *const prof = (PROF && g.prof && static_cast<int>(blockIdx.x) < g.prof_blocks) ? g.prof + kProfSlots * blockIdx.x : nullptr;

    if (PROF && prof && threadIdx.x == 0) prof[13] = static_cast<long long>(global_timer_ns());  // kernel entry

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *const sm = smem_raw + (base - raw);
    const uint32_t bars = base + off_bars;
    volatile int *const abort_flag = reinterpret_cast<volatile int *>(sm + off_tmem_ptr + 4);
    volatile uint32_t *const tmem_slot = reinterpret_cast<volatile uint32_t *>(sm + off_tmem_ptr);

    // Warp-uniform values are broadcast from lane 0 so the compiler can prove them uniform: role
    // dispatch and the role loops then stay convergent code, and addresses, descriptors and
    // coordinates of the TMA / tcgen05 instructions can live in uniform registers.
    const int tid = threadIdx.x;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int lane = tid & 31;
    const int mma_warp = P;
    // A cluster is CG x cl_split CTAs: pairs of consecutive ranks form the tcgen05 groups (CG == 2),
    // the pairs (or single CTAs) of a cluster take the K slices of one tile (cl_split > 1).
    const bool clustered = (CG == 2) || c.cl_split > 1;
    const uint32_t ctarank = clustered ? __shfl_sync(0xffffffffu, cluster_ctarank(), 0) : 0u;
    const uint32_t rank = (CG == 2) ? (ctarank & 1u) : 0u;            // rank inside the pair
    const uint32_t leader_cta = (CG == 2) ? (ctarank & ~1u) : ctarank;  // cluster rank of the pair's leader
    const uint16_t pair_mask = static_cast<uint16_t>(3u << leader_cta);
    c.cl_seg_begin = 0;
    c.cl_seg_end = c.num_segs;
    if (c.cl_split > 1) {
        c.cl_rank = static_cast<int>(ctarank) / CG;
        c.cl_seg_begin = static_cast<int>(static_cast<unsigned>(c.cl_rank) * static_cast<unsigned>(c.num_segs) / static_cast<unsigned>(c.cl_split));
        c.cl_seg_end = static_cast<int>(static_cast<unsigned>(c.cl_rank + 1) * static_cast<unsigned>(c.num_segs) / static_cast<unsigned>(c.cl_split));
    }
    const int group = static_cast<int>(blockIdx.x) / (CG * c.cl_split);   // CTAs that share a tile share a group
    const int num_groups = static_cast<int>(gridDim.x) / (CG * c.cl_split);

    // Barrier map, per stage: [full A x a_bars][full B x b_bars][empty A][pad x (a_bars-1)][empty B x b_bars];
    // after the stages: tmem_full[2], tmem_empty[2].
    const uint32_t stage_bar_bytes = 8u * 2u * static_cast<uint32_t>(c.a_bars + c.b_bars);
    const uint32_t full_b_off = 8u * static_cast<uint32_t>(c.a_bars);
    const uint32_t empty_a_off = 8u * static_cast<uint32_t>(c.a_bars + c.b_bars);
    const uint32_t empty_b_off = 8u * static_cast<uint32_t>(2 * c.a_bars + c.b_bars);
    const uint32_t tmem_full0 = bars + static_cast<uint32_t>(c.stages) * stage_bar_bytes;
    const uint32_t tmem_empty0 = tmem_full0 + 16u;
    const uint32_t part_full = tmem_full0 + 32u;   // cluster reduce: every slice of the tile sits in its CTA's shared memory
    const uint32_t part_empty = tmem_full0 + 40u;  // ... and every CTA of the cluster has read this CTA's slice

    // Barrier initialisation, one barrier per thread (a single thread took over a microsecond for
    // the 26 barriers of a five-stage ring). Per stage: the full barriers of A expect both issuing
    // warps when A and B^T share one barrier; everything else expects one arrival.
    {
        const int per_stage = 2 * (c.a_bars + c.b_bars);
        const int ring = c.stages * per_stage;
        const bool shared_full = (c.a_bars == 1 && c.b_bars == 1 && P > 1);
        for (int i = tid; i < ring + 6; i += static_cast<int>(blockDim.x)) {
            uint32_t count = 1;
            if (i < ring) {
                if (shared_full && (i % per_stage) == 0) count = 2;
            } else {
                const int j = i - ring;  // tmem_full[2], tmem_empty[2], part_full, part_empty
                if (j == 2 || j == 3) count = static_cast<uint32_t>(c.epi_warps * CG);
                if (j >= 4) count = static_cast<uint32_t>(c.epi_warps * c.cl_split);
            }
            mbar_init(bars + 8u * static_cast<uint32_t>(i), count);
            fence_mbar_init();
        }
        if (tid == 0) {
            *abort_flag = 0;
            B200_TL(16);
        }
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&g.map_a);
        tma_prefetch_desc(&g.map_b);
        if (c.epi_mode) tma_prefetch_desc(&g.map_d);
    }
    if (warp == mma_warp) {
        tmem_alloc<CG>(base + off_tmem_ptr, static_cast<uint32_t>(tmem_cols));
        tmem_relinquish<CG>();
        if (lane == 0) B200_TL(17);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (clustered) {
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after_sync();
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);
    if (g.overlap_launch) {
        // Everything above touched only this CTA's shared and tensor memory, so it may run while the
        // previous kernel of the stream is still finishing. Let the next kernel do the same, then wait
        // for the previous one before the first global access (operand loads, C, D, workspace).
        griddep_launch_dependents();
        griddep_wait();
    }

    if (PROF && prof && tid == 0) prof[14] = static_cast<long long>(global_timer_ns());  // set-up done, roles start

    const int b_box_rows = c.chunk_n / CG;  // B^T rows per TMA box in this CTA

    // With one barrier per operand per stage (no sub-tiles) A and B^T share one full and one
    // empty barrier: one wait and one commit per stage for the MMA warp.
    const bool merged = (c.a_bars == 1 && c.b_bars == 1);

    if (SIMPLE && warp < P) {
        // ------------------------------------------------------------------ producers, lean form
        // One full and one empty barrier per stage. With one producer warp it issues the A and
        // the B^T boxes; with more, warp 0 issues A and warp 1 issues B^T (the reference's split,
        // port_1.cu:197) and both arm the same full barrier. The loop carries running addresses,
        // so one stage costs a wait, an arm and one copy instruction per box.
        const bool do_a = (P == 1) || (warp == 0);
        const bool do_b = (P == 1) || (warp == 1);
        if (do_a || do_b) {
            const bool issuer = elect_one();
            const uint32_t a_kb_bytes = static_cast<uint32_t>(c.cta_rows_a * kSwizzleBytes);
            const uint32_t b_kb_bytes = static_cast<uint32_t>((c.tile_n / CG) * kSwizzleBytes);
            const uint32_t my_bytes = static_cast<uint32_t>(c.kblocks * CG) * ((do_a ? a_kb_bytes : 0u) + (do_b ? b_kb_bytes : 0u));
            const uint32_t bars_leader = (CG == 2) ? __shfl_sync(0xffffffffu, mapa_shared(bars, leader_cta), 0) : bars;
            const bool arm = issuer && rank == 0;
            const int hint = g.l2_hint;
            // the hint names the caller's operands; with swapped roles map_a holds B^T and map_b holds A
            const int kind_a = hint >= 1 ? 2 : 0;
            const int kind_b = hint == 1 ? 1 : (hint == 3 ? 2 : 0);
            const uint64_t pol_a = l2_policy(swap_ab ? kind_b : kind_a);
            const uint64_t pol_b = l2_policy(swap_ab ? kind_a : kind_b);
            const bool issue_a = issuer && do_a && !(dbg & 2);
            const bool issue_b = issuer && do_b && !(dbg & 2);
            if (lane == 0 && warp == 0) B200_TL(27);
            int s = 0;
            uint32_t ph = 0, it = 0;
            uint32_t stage = base, sb = bars, sbl = bars_leader;
            bool ok = true;
            int tile_no = 0;
            const bool k_serpentine = g.k_order == 1;
            long long t_wait = 0;
            const long long t_begin = PROF ? clock64() : 0;
            Walk walk;
            walk_init(c, walk, group);
            Unit w;
            while (ok && walk_next(c, walk, num_groups, w)) {
                const int a_row = w.m0 + static_cast<int>(rank) * c.cta_rows_a;
                const int b_row = w.n0 + static_cast<int>(rank) * (c.tile_n / CG);
                // Serpentine K: every other tile of this CTA walks its K segments downwards, so the
                // operand panels a wave touched last are the first the next wave asks for (they are
                // still in L2). The MMA warp is indifferent: it sums whatever the stages bring.
                const int seg_k_elems = c.kblocks * kBoxK;
                const bool down = k_serpentine && (tile_no & 1);
                int k = (down ? w.seg_end - 1 : w.seg_begin) * seg_k_elems;
                const int k_next = down ? -2 * seg_k_elems : 0;   // after a segment k has advanced by one segment
                if (tile_no == 0 && lane == 0 && warp == 0) B200_TL(28);
                ++tile_no;
                for (int seg = w.seg_begin; seg < w.seg_end; ++seg) {
                    const long long tw = PROF ? clock64() : 0;
                    ok = wait_all(sb + empty_a_off, ph ^ 1u, c.budget, abort_flag, 100 + s);
                    if (PROF) t_wait += clock64() - tw;
                    if (!ok) break;
                    if (arm) mbar_arrive_expect_tx(sb, (dbg & 2) ? 0u : my_bytes);
                    if (it == 0 && lane == 0 && warp == 0) B200_TL(19);
                    uint32_t da = stage, db = stage + static_cast<uint32_t>(c.a_stage_bytes);
                    for (int kb = 0; kb < c.kblocks; ++kb) {
                        if constexpr (CG == 2) {
                            if (issue_a) tma_load_2d_pair_hint(da, &g.map_a, sbl, k, a_row, pol_a);
                            if (issue_b) tma_load_2d_pair_hint(db, &g.map_b, sbl, k, b_row, pol_b);
                        } else {
                            if (issue_a) tma_load_2d_hint(da, &g.map_a, sb, k, a_row, pol_a);
                            if (issue_b) tma_load_2d_hint(db, &g.map_b, sb, k, b_row, pol_b);
                        }
                        da += a_kb_bytes;
                        db += b_kb_bytes;
                        k += kBoxK;
                    }
                    ++it;
                    k += k_next;
                    stage += static_cast<uint32_t>(c.stage_bytes);
                    sb += stage_bar_bytes;
                    sbl += stage_bar_bytes;
                    if (++s == c.stages) {
                        s = 0;
                        ph ^= 1u;
                        stage = base;
                        sb = bars;
                        sbl = bars_leader;
                    }
                }
            }
            if (PROF && prof && lane == 0) {
                prof[warp == 0 ? 0 : 3] = t_wait;
                prof[warp == 0 ? 1 : 4] = clock64() - t_begin;
                prof[warp == 0 ? 2 : 5] = it;
            }
        }
    } else if (SIMPLE && warp == mma_warp) {
        // ------------------------------------------------------------------ MMA issue, lean form
        if (rank == 0) {
            const bool issuer = elect_one();
            const bool issue = issuer && !(dbg & 1);
            const uint64_t a_desc0 = umma_desc_sw128(base);
            const uint64_t b_desc0 = umma_desc_sw128(base + static_cast<uint32_t>(c.a_stage_bytes));
            const uint64_t stage_step = static_cast<uint64_t>(c.stage_bytes >> 4);
            const uint64_t a_kb_step = static_cast<uint64_t>((c.cta_rows_a * kSwizzleBytes) >> 4);
            const uint64_t b_kb_step = static_cast<uint64_t>(((c.tile_n / CG) * kSwizzleBytes) >> 4);
            const uint32_t idesc = c.idesc_res;
            const uint64_t atom_step = static_cast<uint64_t>((c.mma_m * kSwizzleBytes) >> 4);   // second atom: the next rows of the A box
            const uint32_t atom_cols = static_cast<uint32_t>(c.tile_n);
            const bool two_atoms = g.atoms == 2;
            const bool two_slots = 2 * c.acc_cols <= 512;   // else one accumulator slot: the next tile's MMAs wait for the drain
            int s = 0;
            uint32_t ph = 0, it = 0, tl = 0;
            uint32_t sb = bars;
            uint64_t a_desc = a_desc0, b_desc = b_desc0;
            bool ok = true;
            long long t_full = 0, t_acc = 0;
            const long long t_begin = PROF ? clock64() : 0;
            Walk walk;
            walk_init(c, walk, group);
            Unit w;
            for (; ok && walk_next(c, walk, num_groups, w); ++tl) {
                const uint32_t acc = two_slots ? (tl & 1u) : 0u;
                const uint32_t aph = two_slots ? ((tl >> 1) & 1u) : (tl & 1u);
                const long long ta = PROF ? clock64() : 0;
                ok = wait_all(tmem_empty0 + 8u * acc, aph ^ 1u, c.budget, abort_flag, 300 + static_cast<int>(acc));
                if (PROF) t_acc += clock64() - ta;
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_addr = tmem_base + acc * static_cast<uint32_t>(c.acc_cols);
                uint32_t accumulate = 0;
                int seg = w.seg_begin;
                if (two_atoms && !two_slots) {
                    // One accumulator slot, two atoms: the draining warps hand back the upper atom's columns first. Its
                    // MMAs for as many stages as the ring holds are issued while the lower atom is still being drained;
                    // the lower atom's MMAs for those stages follow when its columns are free, and release the stages.
                    const int ahead = min(c.stages, w.seg_end - w.seg_begin);
                    {
                        int s1 = s;
                        uint32_t ph1 = ph, sb1 = sb, first = 0;
                        uint64_t a1 = a_desc, b1 = b_desc;
                        for (int j = 0; j < ahead; ++j) {
                            const long long tf = PROF ? clock64() : 0;
                            ok = wait_all(sb1, ph1, c.budget, abort_flag, 400 + s1);
                            if (PROF) t_full += clock64() - tf;
                            if (!ok) break;
                            tc_fence_after_sync();
                            uint64_t da = a1, db = b1;
                            for (int kb = 0; kb < c.kblocks; ++kb) {
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    if (issue) umma_f16<CG>(d_addr, da + static_cast<uint64_t>(2 * i), db + static_cast<uint64_t>(2 * i), idesc, first);
                                    first = 1;
                                }
                                da += a_kb_step;
                                db += b_kb_step;
                            }
                            a1 += stage_step;
                            b1 += stage_step;
                            sb1 += stage_bar_bytes;
                            if (++s1 == c.stages) {
                                s1 = 0;
                                ph1 ^= 1u;
                                a1 = a_desc0;
                                b1 = b_desc0;
                                sb1 = bars;
                            }
                        }
                    }
                    if (!ok) break;
                    const long long ta1 = PROF ? clock64() : 0;
                    ok = wait_all(tmem_empty0 + 8u, aph ^ 1u, c.budget, abort_flag, 301);   // the lower atom's columns
                    if (PROF) t_acc += clock64() - ta1;
                    if (!ok) break;
                    tc_fence_after_sync();
                    uint32_t first = 0;
                    for (int j = 0; j < ahead; ++j, ++seg) {
                        uint64_t da = a_desc + atom_step, db = b_desc;
                        for (int kb = 0; kb < c.kblocks; ++kb) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                if (issue) umma_f16<CG>(d_addr + atom_cols, da + static_cast<uint64_t>(2 * i), db + static_cast<uint64_t>(2 * i), idesc, first);
                                first = 1;
                            }
                            da += a_kb_step;
                            db += b_kb_step;
                        }
                        if (issuer) commit_to<CG>(sb + empty_a_off, pair_mask);
                        ++it;
                        a_desc += stage_step;
                        b_desc += stage_step;
                        sb += stage_bar_bytes;
                        if (++s == c.stages) {
                            s = 0;
                            ph ^= 1u;
                            a_desc = a_desc0;
                            b_desc = b_desc0;
                            sb = bars;
                        }
                    }
                    accumulate = 1;
                }
                for (; seg < w.seg_end; ++seg) {
                    const long long tf = PROF ? clock64() : 0;
                    ok = wait_all(sb, ph, c.budget, abort_flag, 400 + s);
                    if (PROF) t_full += clock64() - tf;
                    if (!ok) break;
                    if (it == 0 && lane == 0) B200_TL(20);
                    tc_fence_after_sync();
                    uint64_t da = a_desc, db = b_desc;
                    if (!two_atoms) {
                        for (int kb = 0; kb < c.kblocks; ++kb) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                // +32 bytes per 16-element K step inside the 128-byte swizzle row
                                if (issue) umma_f16<CG>(d_addr, da + static_cast<uint64_t>(2 * i), db + static_cast<uint64_t>(2 * i), idesc, accumulate);
                                accumulate = 1;
                            }
                            da += a_kb_step;
                            db += b_kb_step;
                        }
                    } else {
                        // two 128-row atoms of A against the same B^T rows: accumulators side by side
                        for (int kb = 0; kb < c.kblocks; ++kb) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                if (issue) {
                                    umma_f16<CG>(d_addr, da + static_cast<uint64_t>(2 * i), db + static_cast<uint64_t>(2 * i), idesc, accumulate);
                                    umma_f16<CG>(d_addr + atom_cols, da + atom_step + static_cast<uint64_t>(2 * i), db + static_cast<uint64_t>(2 * i), idesc, accumulate);
                                }
                                accumulate = 1;
                            }
                            da += a_kb_step;
                            db += b_kb_step;
                        }
                    }
                    if (issuer) commit_to<CG>(sb + empty_a_off, pair_mask);
                    ++it;
                    a_desc += stage_step;
                    b_desc += stage_step;
                    sb += stage_bar_bytes;
                    if (++s == c.stages) {
                        s = 0;
                        ph ^= 1u;
                        a_desc = a_desc0;
                        b_desc = b_desc0;
                        sb = bars;
                    }
                }
                if (!ok) break;
                if (issuer) commit_to<CG>(tmem_full0 + 8u * acc, pair_mask);
                if (lane == 0) B200_TL(21);
            }
            if (PROF && prof && lane == 0) {
                prof[6] = t_full;
                prof[7] = t_acc;
                prof[8] = clock64() - t_begin;
                prof[9] = it;
            }
        }
        __syncwarp();
    } else if (warp < P) {
        // ------------------------------------------------------------------ producers, general form
        // Sub-tile barriers (shift synchronisation): the A stage buffer is loaded in row boxes, the
        // B^T buffer in column sub-tiles, each group with its own full barrier; the first a_priv /
        // b_priv groups are private, the rest share a residual barrier. Same lean structure as
        // above: converged warp, one elected issuing lane, running addresses.
        const bool do_a = (P == 1) || (warp == 0);
        const bool do_b = (P == 1) || (warp == 1);
        if (do_a || do_b) {
            const bool issuer = elect_one();
            const bool arm = issuer && rank == 0;
            const bool issue = issuer && !(dbg & 2);
            const uint32_t bars_leader = (CG == 2) ? __shfl_sync(0xffffffffu, mapa_shared(bars, leader_cta), 0) : bars;
            const uint32_t a_box_bytes = static_cast<uint32_t>(c.a_box_rows * kSwizzleBytes);
            const uint32_t a_kb_bytes = static_cast<uint32_t>(c.cta_rows_a * kSwizzleBytes);
            const uint32_t a_priv_tx = (dbg & 2) ? 0u : static_cast<uint32_t>(c.kblocks * CG) * a_box_bytes;
            const uint32_t a_res_tx = a_priv_tx * static_cast<uint32_t>(c.a_boxes - c.a_priv);
            const uint32_t b_box_bytes = static_cast<uint32_t>(b_box_rows * kSwizzleBytes);
            const uint32_t b_priv_tx = (dbg & 2) ? 0u : static_cast<uint32_t>(c.kblocks * c.chunk_n * kSwizzleBytes);
            const uint32_t b_res_tx = b_priv_tx * static_cast<uint32_t>(c.b_res_chunks);
            const uint32_t b_sub_bytes = b_box_bytes * static_cast<uint32_t>(c.kblocks);  // one private sub-tile in this CTA
            const uint32_t b_all_tx = (dbg & 2) ? 0u : static_cast<uint32_t>(c.kblocks * c.tile_n * kSwizzleBytes);
            int s = 0;
            uint32_t ph = 0, it = 0;
            uint32_t stage = base, sb = bars, sbl = bars_leader;
            bool ok = true;
            long long t_wait = 0;
            const long long t_begin = PROF ? clock64() : 0;
            Walk walk;
            walk_init(c, walk, group);
            Unit w;
            while (ok && walk_next(c, walk, num_groups, w)) {
                const int a_row = w.m0 + static_cast<int>(rank) * c.cta_rows_a;
                int k = w.seg_begin * c.kblocks * kBoxK;
                for (int seg = w.seg_begin; ok && seg < w.seg_end; ++seg) {
                    if (do_a) {
                        const long long tw = PROF ? clock64() : 0;
                        ok = wait_all(sb + empty_a_off, ph ^ 1u, c.budget, abort_flag, 100 + s);
                        if (PROF) t_wait += clock64() - tw;
                        if (!ok) break;
                        uint32_t box_dst = stage;
                        int box_row = a_row;
                        for (int j = 0; j < c.a_bars; ++j) {
                            const bool priv = j < c.a_priv;
                            const int nbox = priv ? 1 : c.a_boxes - c.a_priv;
                            uint32_t tx = priv ? a_priv_tx : a_res_tx;
                            if (merged && P == 1) tx += b_all_tx;
                            if (arm) mbar_arrive_expect_tx(sb + 8u * j, tx);
                            const uint32_t bar = ((CG == 2) ? sbl : sb) + 8u * j;
                            uint32_t kb_dst = box_dst;
                            int kk = k;
                            for (int kb = 0; kb < c.kblocks; ++kb) {
                                uint32_t d = kb_dst;
                                int r = box_row;
                                for (int b = 0; b < nbox; ++b) {
                                    if (issue) {
                                        if constexpr (CG == 2) tma_load_2d_pair(d, &g.map_a, bar, kk, r);
                                        else tma_load_2d(d, &g.map_a, bar, kk, r);
                                    }
                                    d += a_box_bytes;
                                    r += c.a_box_rows;
                                }
                                kb_dst += a_kb_bytes;
                                kk += kBoxK;
                            }
                            box_dst += a_box_bytes;
                            box_row += c.a_box_rows;
                        }
                    }
                    if (do_b) {
                        uint32_t sub = stage + static_cast<uint32_t>(c.a_stage_bytes);
                        int sub_row = w.n0;
                        for (int t = 0; t < c.b_bars; ++t) {
                            if (!(merged && do_a)) {  // merged + same warp: the stage was acquired above
                                const long long tw = PROF ? clock64() : 0;
                                ok = wait_all(sb + (merged ? empty_a_off : empty_b_off + 8u * t), ph ^ 1u, c.budget, abort_flag,
                                              200 + s * 32 + t);
                                if (PROF) t_wait += clock64() - tw;
                                if (!ok) break;
                            }
                            const bool priv = t < c.b_priv;
                            const int nbox = priv ? 1 : c.b_res_chunks;       // boxes of b_box_rows rows per K block
                            const uint32_t bar_off = merged ? 0u : full_b_off + 8u * t;
                            if (arm && !(merged && P == 1)) mbar_arrive_expect_tx(sb + bar_off, priv ? b_priv_tx : b_res_tx);
                            const uint32_t bar = ((CG == 2) ? sbl : sb) + bar_off;
                            const int row0 = sub_row + static_cast<int>(rank) * nbox * b_box_rows;
                            uint32_t d = sub;
                            int kk = k;
                            for (int kb = 0; kb < c.kblocks; ++kb) {
                                int r = row0;
                                for (int b = 0; b < nbox; ++b) {
                                    if (issue) {
                                        if constexpr (CG == 2) tma_load_2d_pair(d, &g.map_b, bar, kk, r);
                                        else tma_load_2d(d, &g.map_b, bar, kk, r);
                                    }
                                    d += b_box_bytes;
                                    r += b_box_rows;
                                }
                                kk += kBoxK;
                            }
                            sub += b_sub_bytes;
                            sub_row += c.chunk_n;
                        }
                        if (!ok) break;
                    }
                    ++it;
                    k += c.kblocks * kBoxK;
                    stage += static_cast<uint32_t>(c.stage_bytes);
                    sb += stage_bar_bytes;
                    sbl += stage_bar_bytes;
                    if (++s == c.stages) {
                        s = 0;
                        ph ^= 1u;
                        stage = base;
                        sb = bars;
                        sbl = bars_leader;
                    }
                }
            }
            if (PROF && prof && lane == 0) {
                prof[warp == 0 ? 0 : 3] = t_wait;
                prof[warp == 0 ? 1 : 4] = clock64() - t_begin;
                prof[warp == 0 ? 2 : 5] = it;
            }
        }
    } else if (warp == mma_warp) {
        // ------------------------------------------------------------------ MMA issue, general form
        // One MMA group per B^T sub-tile, in load order: the first sub-tile's MMAs start as soon as
        // A and that sub-tile have landed. Each sub-tile frees its own part of the stage.
        if (rank == 0) {
            const bool issuer = elect_one();
            const bool issue = issuer && !(dbg & 1);
            const uint64_t a_desc0 = umma_desc_sw128(base);
            const uint64_t b_desc0 = umma_desc_sw128(base + static_cast<uint32_t>(c.a_stage_bytes));
            const uint64_t stage_step = static_cast<uint64_t>(c.stage_bytes >> 4);
            const uint64_t a_kb_step = static_cast<uint64_t>((c.cta_rows_a * kSwizzleBytes) >> 4);
            const uint64_t b_box_step = static_cast<uint64_t>((b_box_rows * kSwizzleBytes) >> 4);   // one box of a K block
            const uint64_t b_sub_step = b_box_step * static_cast<uint64_t>(c.kblocks);             // one private sub-tile
            const uint64_t a_half_step = static_cast<uint64_t>((c.mma_m * kSwizzleBytes) >> 4);  // the second atom's rows of a K block
            const int a_halves = g.atoms;
            const bool two_slots = 2 * c.acc_cols <= 512;
            long long n_early = 0;
            int s = 0;
            uint32_t ph = 0, it = 0, tl = 0;
            uint32_t sb = bars;
            uint64_t a_desc = a_desc0, b_desc = b_desc0;
            bool ok = true;
            long long t_full = 0, t_acc = 0;
            const long long t_begin = PROF ? clock64() : 0;
            Walk walk;
            walk_init(c, walk, group);
            Unit w;
            for (; ok && walk_next(c, walk, num_groups, w); ++tl) {
                const uint32_t acc = two_slots ? (tl & 1u) : 0u;
                const uint32_t aph = two_slots ? ((tl >> 1) & 1u) : (tl & 1u);
                const long long ta = PROF ? clock64() : 0;
                ok = wait_all(tmem_empty0 + 8u * acc, aph ^ 1u, c.budget, abort_flag, 300 + static_cast<int>(acc));
                if (PROF) t_acc += clock64() - ta;
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_base = tmem_base + acc * static_cast<uint32_t>(c.acc_cols);
                uint32_t later_seg = 0;
                for (int seg = w.seg_begin; ok && seg < w.seg_end; ++seg) {
                    // The A side of the reference's shift synchronisation (port_1.cu:406-433: a consumer waits per
                    // fragment row and starts on the first rows while later ones are still being loaded): with two
                    // 64-row atoms per tile (a_halves == 2) the upper atom's MMAs wait only for the barriers of the
                    // row boxes of rows 0-63 and are issued before the lower rows have landed; the lower atom follows
                    // when its boxes are there. With one 128-row atom every A barrier is waited first.
                    int a_waited = 0;     // A barriers of this stage already waited for
                    for (int mh = 0; ok && mh < a_halves; ++mh) {
                        const long long tf = PROF ? clock64() : 0;
                        // barriers that cover this half's row boxes: box b -> barrier min(b, a_priv)
                        const int last_box = (a_halves == 2) ? ((mh + 1) * c.a_boxes / 2 - 1) : (c.a_boxes - 1);
                        const int need = min(last_box, c.a_priv) + 1 < c.a_bars ? min(last_box, c.a_priv) + 1 : c.a_bars;
                        for (; ok && a_waited < need; ++a_waited)
                            ok = wait_all(sb + 8u * a_waited, ph, c.budget, abort_flag, 400 + s * 32 + a_waited);
                        if (PROF) t_full += clock64() - tf;
                        if (!ok) break;
                        if (PROF && a_halves == 2 && mh == 0 && a_waited < c.a_bars) {
                            // are the last rows of A still on their way as the upper atom's first MMA goes out?
                            const bool landed = mbar_try_wait(sb + 8u * static_cast<uint32_t>(c.a_bars - 1), ph);
                            if (!__all_sync(0xffffffffu, landed)) ++n_early;
                        }
                        uint64_t sub_desc = b_desc;
                        uint32_t d_addr = d_base + static_cast<uint32_t>(mh * c.tile_n);
                        for (int t = 0; t < c.b_bars; ++t) {
                            if (!merged && mh == 0) {
                                const long long tb = PROF ? clock64() : 0;
                                ok = wait_all(sb + full_b_off + 8u * t, ph, c.budget, abort_flag, 500 + s * 32 + t);
                                if (PROF) t_full += clock64() - tb;
                                if (!ok) break;
                            }
                            tc_fence_after_sync();
                            const bool priv = t < c.b_priv;
                            const uint32_t idesc = priv ? c.idesc_chunk : c.idesc_res;
                            const uint64_t b_kb_step = priv ? b_box_step : b_box_step * static_cast<uint64_t>(c.b_res_chunks);
                            uint64_t da = a_desc + static_cast<uint64_t>(mh) * a_half_step, db = sub_desc;
                            for (int kb = 0; kb < c.kblocks; ++kb) {
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    // +32 bytes per 16-element K step inside the 128-byte swizzle row
                                    if (issue)
                                        umma_f16<CG>(d_addr, da + static_cast<uint64_t>(2 * i), db + static_cast<uint64_t>(2 * i), idesc,
                                                     (later_seg | static_cast<uint32_t>(kb) | static_cast<uint32_t>(i)) ? 1u : 0u);
                                }
                                da += a_kb_step;
                                db += b_kb_step;
                            }
                            // a B^T sub-tile is free when the last atom has read it
                            if (!merged && issuer && mh == a_halves - 1) commit_to<CG>(sb + empty_b_off + 8u * t, pair_mask);
                            sub_desc += b_sub_step;
                            d_addr += static_cast<uint32_t>(c.chunk_n);
                        }
                    }
                    if (!ok) break;
                    if (issuer) commit_to<CG>(sb + empty_a_off, pair_mask);
                    later_seg = 1;
                    ++it;
                    a_desc += stage_step;
                    b_desc += stage_step;
                    sb += stage_bar_bytes;
                    if (++s == c.stages) {
                        s = 0;
                        ph ^= 1u;
                        a_desc = a_desc0;
                        b_desc = b_desc0;
                        sb = bars;
                    }
                }
                if (!ok) break;
                if (issuer) commit_to<CG>(tmem_full0 + 8u * acc, pair_mask);
            }
            if (PROF && prof && lane == 0) {
                prof[6] = t_full;
                prof[7] = t_acc;
                prof[8] = clock64() - t_begin;
                prof[9] = it;
                prof[kEarlySlot] = n_early;
                prof[kEarlySlot + 1] = it;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue
        const int e = warp - (P + 1);          // 0 .. epi_warps-1
        const int a_halves = g.atoms;   // 64-row atoms (a_split) or 128-row atoms (the tall pair): mma_m rows each
        const int q = warp & 3;                // TMEM lane quarter this warp may read
        const int halves = c.epi_warps / 4;    // 1 or 2 warps per quarter
        const int half = e / 4;
        int col_begin = 0, col_end = c.tile_n;
        if (halves == 2) {
            const int mid = ((c.tile_n / 2 + 31) / 32) * 32;
            col_begin = half ? min(mid, c.tile_n) : 0;
            col_end = half ? c.tile_n : min(mid, c.tile_n);
        }
        const uint32_t tmem_empty_leader = (CG == 2) ? mapa_shared(tmem_empty0, leader_cta) : tmem_empty0;
        const uint32_t two_bufs = g.epi_bufs == 2 ? 1u : 0u;   // 1: two staging boxes per warp, alternating; 0: one
        const uint32_t epi_buf = base + static_cast<uint32_t>(off_epi) + static_cast<uint32_t>(e) * (4096u << two_bufs);
        // row of the tile this thread drains: 128-row atoms map row r to lane r; 64-row atoms use
        // lanes 0-15 of each quarter (row 16 * quarter + lane).
        const int row_in_cta = (c.mma_m == 128) ? (q * 32 + lane) : (q * 16 + (lane & 15));
        const bool lane_has_row = (c.mma_m == 128) || (lane < 16);
        const bool to_partial = c.split_k > 1;
        const float alpha = (to_partial || push_world > 0) ? 1.0f : g_alpha;
        const float beta = (to_partial || push_world > 0) ? 0.0f : g_beta;
        uint32_t tl = 0;
        uint32_t store_idx = 0;
        // D is written once and not read again by this launch: when it is larger than the L2 can keep anyway, its
        // lines are marked to leave first, so that they do not push out operand panels the next tiles re-read
        const uint64_t d_policy = l2_policy(g.d_stream ? 1 : 0);
        bool ok = true;
        long long t_tfull = 0;
        const long long t_begin = clock64();
        Walk walk;
        walk_init(c, walk, group);
        Unit w;
        for (; ok && walk_next(c, walk, num_groups, w); ++tl) {
            const bool two_slots = 2 * c.acc_cols <= 512;
            const uint32_t acc = two_slots ? (tl & 1u) : 0u;
            const uint32_t aph = two_slots ? ((tl >> 1) & 1u) : (tl & 1u);
            const long long te = prof ? clock64() : 0;
            ok = wait_all(tmem_full0 + 8u * acc, aph, c.budget, abort_flag, 600 + static_cast<int>(acc));
            if (prof) t_tfull += clock64() - te;
            if (!ok) break;
            if (tl == 0 && e == 0 && lane == 0) B200_TL(22);
            if (e == 0 && lane == 0) B200_TL(26);   // last tile: accumulator ready
            tc_fence_after_sync();
            const int row = w.m0 + static_cast<int>(rank) * c.cta_rows_a + row_in_cta;
            const bool row_ok = lane_has_row && row < c.M;
            float *out = to_partial ? g_partial + static_cast<size_t>(w.slice) * c.M * c.N : gD;
            size_t row_off = static_cast<size_t>(row) * (to_partial ? c.N : ld_cd) + w.n0;
            if (push_world > 0) {
                // the 128 rows this CTA drains belong to one owner (rows per owner is a multiple of 128)
                const int cta_row0 = w.m0 + static_cast<int>(rank) * c.cta_rows_a;
                const int owner = cta_row0 / push_rows;
                out = g.push_slot[owner];
                row_off = (static_cast<size_t>(push_rank) * push_rows + static_cast<size_t>(row - owner * push_rows)) * c.N + w.n0;
            }
            // alpha * acc + beta * C is evaluated everywhere as fma(beta, C, round(alpha * acc)), written with the intrinsic so
            // that every drain path (and every tiling) rounds the same way
            const float a_u = alpha;
            const float b_u = beta;
            const uint32_t t_row = tmem_base + acc * static_cast<uint32_t>(c.acc_cols) + (static_cast<uint32_t>(q * 32) << 16);
            // Tail split. The workspace holds one partial per CTA and slice unit: per 32-lane quarter and 32-column
            // chunk eight groups of [32 lanes] float4 (lane l keeps its columns 4j .. 4j+3 in group j), so a warp
            // stores and re-loads 512 consecutive bytes per instruction, and warp e of the finishing CTA reads
            // exactly what warp e of a peer wrote. The CTA that runs a tile's last slice (kind 1) first waits
            // (bounded) until the CTAs of the earlier slices have stored theirs.
            const int tail_peers = (w.kind == 1) ? c.tail_slices - 1 : 0;
            const int tail_slot = w.slot * CG + static_cast<int>(rank);     // in CTA units
            const int tail_step = c.tail_tiles * CG;                        // from one slice of a tile to the next
            if (w.kind == 1 && !tail_wait_peers(tail_flags, tail_epoch, tail_slot, tail_step, tail_peers, e, c.budget, abort_flag)) {
                ok = false;
                break;
            }
            const uint32_t tail_chunks = static_cast<uint32_t>(c.tile_n + 31) >> 5;
            const uint32_t tail_slot4 = tail_chunks * 1024u;                                // float4 per slot (offsets fit 32 bits)
            const uint32_t tail_lane = static_cast<uint32_t>(q) * tail_chunks * 256u + static_cast<uint32_t>(lane);
            if (c.cl_split > 1) {
                // ---- K slices of this tile live in the CTAs of the cluster (transposed drain only).
                // A: raw accumulator -> this CTA's shared memory as [column][row]; tell every CTA.
                const uint32_t pbuf = base + static_cast<uint32_t>(off_epi);
                ok = wait_all<true>(part_empty, (tl & 1u) ^ 1u, c.budget, abort_flag, 700);  // the peers have read the previous tile
                if (!ok) break;
                for (int c0 = col_begin; c0 < col_end; c0 += 32) {
                    uint32_t r[32];
                    if (col_end - c0 >= 32) {
                        tmem_ld_32x32(t_row + static_cast<uint32_t>(c0), r);
                    } else {
                        uint32_t r16[16];
                        tmem_ld_32x16(t_row + static_cast<uint32_t>(c0), r16);
#pragma unroll
                        for (int j = 0; j < 16; ++j) r[j] = r16[j];
#pragma unroll
                        for (int j = 16; j < 32; ++j) r[j] = 0;
                    }
                    tmem_ld_wait();
                    if (lane_has_row) {
                        // columns beyond the tile are never read back: store the whole 16 or 32 without tests
                        const uint32_t dst = pbuf + static_cast<uint32_t>(c0 * 128 + row_in_cta) * 4u;
                        const bool wide32 = col_end - c0 >= 32;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < 16 || wide32)
                                asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst + static_cast<uint32_t>(j) * 512u), "r"(r[j]) : "memory");
                    }
                }
                // The lanes' shared-memory writes are ordered before the arrivals below by the warp
                // barrier, and the arrivals release at cluster scope (cumulative): no fence needed.
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {                                     // accumulator slot back to the MMA thread
                    if constexpr (CG == 2) mbar_arrive_cluster(tmem_empty_leader + 8u * acc);
                    else mbar_arrive(tmem_empty0 + 8u * acc);
                }
                // the peers of this CTA: the CTA with the same rank in its pair, in every slice of the cluster
                if (lane < c.cl_split && !(dbg & 4)) mbar_arrive_release_cluster(mapa_shared(part_full, static_cast<uint32_t>(lane * CG) + rank));
                if (e == 0 && lane == 0) B200_TL(29);
                // B: when all slices are staged, this CTA sums its share of the tile's columns over the
                // cluster in slice order (the order of the workspace form) and writes D.
                ok = wait_all<true>(part_full, tl & 1u, c.budget, abort_flag, 701);
                if (!ok) break;
                if (e == 0 && lane == 0) B200_TL(30);
                const int per = (c.tile_n + c.cl_split - 1) / c.cl_split;
                const int my_end = min(c.tile_n, (c.cl_rank + 1) * per);
                if (c.mma_m == 128) {
                    // 128-row slices: a warp takes whole columns of the tile (column first + e, then every
                    // epi_warps-th), a lane four consecutive rows, so a column costs one 16-byte remote load
                    // per slice and one 16-byte store per lane (the kernel's M is a multiple of 4).
                    const int row4 = w.m0 + static_cast<int>(rank) * c.cta_rows_a + lane * 4;
                    const bool rows_ok = row4 < c.M;
                    const uint32_t my_rows = pbuf + static_cast<uint32_t>(lane) * 16u;
                    // three columns per round: up to twelve 16-byte remote loads in flight per lane (a round trip through
                    // distributed shared memory takes about a microsecond: the rounds, not the bytes, are the cost)
                    constexpr int kRC = 3;
                    for (int col0 = c.cl_rank * per + e; col0 < my_end; col0 += kRC * c.epi_warps) {
                        float4 sum[kRC];
#pragma unroll
                        for (int cc = 0; cc < kRC; ++cc) sum[cc] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        // slices are added in ascending order, four at a time
                        for (int base4 = 0; base4 < c.cl_split; base4 += 4) {
                            float4 v[kRC][4];
#pragma unroll
                            for (int cc = 0; cc < kRC; ++cc) {
                                const int col = col0 + cc * c.epi_warps;
                                const uint32_t src = my_rows + static_cast<uint32_t>(col) * 512u;
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    if (base4 + i < c.cl_split && col < my_end)
                                        v[cc][i] = ld_shared_cluster_v4(mapa_shared(src, static_cast<uint32_t>((base4 + i) * CG) + rank));
                            }
#pragma unroll
                            for (int cc = 0; cc < kRC; ++cc)
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    if (base4 + i < c.cl_split && col0 + cc * c.epi_warps < my_end) {
                                        sum[cc].x += v[cc][i].x;
                                        sum[cc].y += v[cc][i].y;
                                        sum[cc].z += v[cc][i].z;
                                        sum[cc].w += v[cc][i].w;
                                    }
                        }
#pragma unroll
                        for (int cc = 0; cc < kRC; ++cc) {
                            const int col = col0 + cc * c.epi_warps;
                            const int gcol = w.n0 + col;
                            if (!(rows_ok && col < my_end && gcol < c.N)) continue;
                            const size_t off = static_cast<size_t>(gcol) * static_cast<size_t>(ld_cd) + static_cast<size_t>(row4);
                            float4 val = make_float4(alpha * sum[cc].x, alpha * sum[cc].y, alpha * sum[cc].z, alpha * sum[cc].w);
                            if (out_half) {
                                if (beta != 0.0f) {
                                    const uint2 cv = *reinterpret_cast<const uint2 *>(reinterpret_cast<const __half *>(gC) + off);
                                    const float2 c01 = __half22float2(*reinterpret_cast<const __half2 *>(&cv.x));
                                    const float2 c23 = __half22float2(*reinterpret_cast<const __half2 *>(&cv.y));
                                    val.x = __fmaf_rn(beta, c01.x, val.x);
                                    val.y = __fmaf_rn(beta, c01.y, val.y);
                                    val.z = __fmaf_rn(beta, c23.x, val.z);
                                    val.w = __fmaf_rn(beta, c23.y, val.w);
                                }
                                const __half2 h01 = __floats2half2_rn(val.x, val.y), h23 = __floats2half2_rn(val.z, val.w);
                                uint2 o;
                                o.x = *reinterpret_cast<const uint32_t *>(&h01);
                                o.y = *reinterpret_cast<const uint32_t *>(&h23);
                                *reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(gD) + off) = o;
                            } else {
                                if (beta != 0.0f) {
                                    const float4 cv = __ldg(reinterpret_cast<const float4 *>(gC + off));
                                    val.x = __fmaf_rn(beta, cv.x, val.x);
                                    val.y = __fmaf_rn(beta, cv.y, val.y);
                                    val.z = __fmaf_rn(beta, cv.z, val.z);
                                    val.w = __fmaf_rn(beta, cv.w, val.w);
                                }
                                *reinterpret_cast<float4 *>(gD + off) = val;
                            }
                        }
                    }
                }
                // 64-row slices (16 lanes of a quarter hold rows): a thread per row
                // this thread's row of column 0, as an address in this CTA; mapa turns it into a peer's
                const uint32_t my_row0 = pbuf + static_cast<uint32_t>(row_in_cta) * 4u;
                // two columns per round: their 2 x cl_split remote loads are in flight together
                for (int col0 = c.cl_rank * per + half; c.mma_m != 128 && col0 < my_end; col0 += 2 * halves) {
                    float v[2][8];
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const int col = col0 + cc * halves;
#pragma unroll
                        for (int sl = 0; sl < 8; ++sl)
                            if (sl < c.cl_split && col < my_end)
                                v[cc][sl] = ld_shared_cluster_f32(mapa_shared(my_row0 + static_cast<uint32_t>(col) * 512u, static_cast<uint32_t>(sl * CG) + rank));
                    }
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const int col = col0 + cc * halves;
                        const int gcol = w.n0 + col;
                        if (col < my_end && gcol < c.N && row_ok) {
                            float sum = v[cc][0];
#pragma unroll
                            for (int sl = 1; sl < 8; ++sl)
                                if (sl < c.cl_split) sum += v[cc][sl];
                            const size_t off = static_cast<size_t>(gcol) * static_cast<size_t>(ld_cd) + static_cast<size_t>(row);
                            float val = alpha * sum;
                            if (out_half) {
                                if (beta != 0.0f) val = __fmaf_rn(beta, __half2float(reinterpret_cast<const __half *>(gC)[off]), val);
                                reinterpret_cast<__half *>(gD)[off] = __float2half_rn(val);
                            } else {
                                if (beta != 0.0f) val = __fmaf_rn(beta, __ldg(gC + off), val);
                                gD[off] = val;
                            }
                        }
                    }
                }
                __syncwarp();
                if (e == 0 && lane == 0) B200_TL(31);
                if (lane < c.cl_split && !(dbg & 8)) mbar_arrive_release_cluster(mapa_shared(part_empty, static_cast<uint32_t>(lane * CG) + rank));
                continue;
            }
            // With two 64-row atoms per tile the drain below runs once per atom: the lower atom's accumulator sits
            // tile_n columns further in tensor memory and its rows 64 further in D (the names of the per-row
            // values are re-declared for the atom, so the drain code is the one-atom code).
            const int row_atom0 = row;
            const size_t row_off_atom0 = row_off;
            const uint32_t t_row_atom0 = t_row;
            // One accumulator slot shared by two atoms: the upper atom's columns go back to the MMA thread as soon as
            // they are drained (barrier 0), the lower atom's at the end of the tile (barrier 1).
            const bool atom_release = a_halves == 2 && !two_slots;
            auto upper_atom_drained = [&]() {
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (CG == 2) mbar_arrive_cluster(tmem_empty_leader);
                    else mbar_arrive(tmem_empty0);
                }
            };
            for (int mh = 0; mh < a_halves; ++mh) {
                const int row = row_atom0 + mh * c.mma_m;
                const bool row_ok = lane_has_row && row < c.M;
                const size_t row_off = row_off_atom0 + static_cast<size_t>(mh * c.mma_m) * static_cast<size_t>(ld_cd);
                const uint32_t t_row = t_row_atom0 + static_cast<uint32_t>(mh * c.tile_n);
                if (w.kind == 0 && tail_peers == 0 && c.epi_mode == 1 && b_u == 0.0f && ((col_end - col_begin) & 31) == 0 && w.n0 + col_end <= c.N) {
                    // ---- The common drain: a whole tile, beta = 0, fp32 D through TMA stores, full 32-column boxes. The same steps
                    // as the general loop below, with the tensor-memory load of the next box issued as soon as this
                    // box's registers have been staged, so that it overlaps the fence, the warp barrier and the store.
                    uint32_t r[32];
                    tmem_ld_32x32(t_row + static_cast<uint32_t>(col_begin), r);
                    const uint32_t my_x = static_cast<uint32_t>(lane & 7);
                    int d_col = w.n0 + col_begin;
                    for (int c0 = col_begin; c0 < col_end; c0 += 32, d_col += 32) {
                        tmem_ld_wait();
                        const uint32_t buf = epi_buf + (store_idx & two_bufs) * 4096u;
                        if (lane == 0) {   // the box stored two steps ago (one step ago with a single box) has been read
                            if (two_bufs) tma_store_wait_read<1>();
                            else tma_store_wait_read<0>();
                        }
                        __syncwarp();
                        const uint32_t my_row = buf + static_cast<uint32_t>(lane) * 128u;
                        if (a_u == 1.0f) {
    #pragma unroll
                            for (int j = 0; j < 8; ++j)
                                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + ((static_cast<uint32_t>(j) ^ my_x) << 4)),
                                             "r"(r[4 * j + 0]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3])
                                             : "memory");
                        } else {
    #pragma unroll
                            for (int j = 0; j < 8; ++j)
                                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + ((static_cast<uint32_t>(j) ^ my_x) << 4)),
                                             "f"(a_u * __uint_as_float(r[4 * j + 0])), "f"(a_u * __uint_as_float(r[4 * j + 1])),
                                             "f"(a_u * __uint_as_float(r[4 * j + 2])), "f"(a_u * __uint_as_float(r[4 * j + 3]))
                                             : "memory");
                        }
                        if (c0 + 32 < col_end) tmem_ld_32x32(t_row + static_cast<uint32_t>(c0 + 32), r);
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d_hint(&g.map_d, buf, d_col, row - lane, d_policy);   // the first of this warp's 32 rows
                            tma_store_commit();
                        }
                        ++store_idx;
                    }
                    if (atom_release && mh == 0) upper_atom_drained();
                    continue;
                }
                for (int c0 = col_begin; c0 < col_end; c0 += 32) {
                    if (w.n0 + c0 >= c.N) break;  // ragged last tile column: nothing of D beyond N
                    uint32_t r[32];
                    const bool wide = (col_end - c0) >= 32;
                    float4 part[8];
                    if (tail_peers > 0) {
                        // The earlier slices' partials of this chunk, summed in ascending K order (this, the last slice, is
                        // added below). Eight independent 16-byte loads per lane and slice are in flight at once, and the
                        // first batch is issued ahead of the tensor-memory load; .cg: other SMs wrote them.
                        const float4 *src = reinterpret_cast<const float4 *>(g_partial) +
                                            (static_cast<uint32_t>(tail_slot) * tail_slot4 + tail_lane + static_cast<uint32_t>(c0 >> 5) * 256u);
                        const uint32_t step4 = static_cast<uint32_t>(tail_step) * tail_slot4;
    #pragma unroll
                        for (int j = 0; j < 8; ++j) part[j] = __ldcg(src + j * 32);
    #pragma unroll 1
                        for (int i = 1; i < tail_peers; ++i) {
                            float4 v[8];
    #pragma unroll
                            for (int j = 0; j < 8; ++j) v[j] = __ldcg(src + i * step4 + j * 32);
    #pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                part[j].x += v[j].x;
                                part[j].y += v[j].y;
                                part[j].z += v[j].z;
                                part[j].w += v[j].w;
                            }
                        }
                    }
                    if (wide) {
                        tmem_ld_32x32(t_row + static_cast<uint32_t>(c0), r);
                    } else {
                        uint32_t r16[16];
                        tmem_ld_32x16(t_row + static_cast<uint32_t>(c0), r16);
    #pragma unroll
                        for (int j = 0; j < 16; ++j) r[j] = r16[j];
    #pragma unroll
                        for (int j = 16; j < 32; ++j) r[j] = 0;
                    }
                    tmem_ld_wait();
                    if (e == 0 && lane == 0) B200_TL(18);
                    const int nvec = wide ? 8 : 4;
                    if (w.kind == 2) {
                        // raw partial of this chunk into this unit's slot (a 16-column last chunk stores its zero padding too)
                        float4 *dst = reinterpret_cast<float4 *>(g_partial) +
                                      (static_cast<uint32_t>(tail_slot) * tail_slot4 + tail_lane + static_cast<uint32_t>(c0 >> 5) * 256u);
    #pragma unroll
                        for (int j = 0; j < 8; ++j)
                            dst[j * 32] = make_float4(__uint_as_float(r[4 * j + 0]), __uint_as_float(r[4 * j + 1]),
                                                      __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                        continue;
                    }
                    if (tail_peers > 0) {
    #pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            r[4 * j + 0] = __float_as_uint(part[j].x + __uint_as_float(r[4 * j + 0]));
                            r[4 * j + 1] = __float_as_uint(part[j].y + __uint_as_float(r[4 * j + 1]));
                            r[4 * j + 2] = __float_as_uint(part[j].z + __uint_as_float(r[4 * j + 2]));
                            r[4 * j + 3] = __float_as_uint(part[j].w + __uint_as_float(r[4 * j + 3]));
                        }
                    }
                    if (swap_ab) {
                        // Transposed drain: this thread's row is a column of D and register j its row
                        // w.n0 + c0 + j, so for every j the 32 lanes store 32 consecutive floats. The
                        // pointers advance by one pitch per register: a handful of instructions per store
                        // (the epilogue warps run alone on their schedulers, every instruction shows).
                        if (row_ok) {
                            const size_t pitch = to_partial ? static_cast<size_t>(c.M) : static_cast<size_t>(ld_cd);
                            const size_t off0 = static_cast<size_t>(w.n0 + c0) * pitch + static_cast<size_t>(row);
                            float *dst = out + off0;
                            const float *csrc = gC + off0;
                            const int valid = min(4 * nvec, c.N - (w.n0 + c0));
                            if (out_half) {
                                __half *dst16 = reinterpret_cast<__half *>(gD) + off0;
                                const __half *c16 = reinterpret_cast<const __half *>(gC) + off0;
    #pragma unroll
                                for (int j = 0; j < 32; ++j) {
                                    if (j < 16 || wide) {
                                        if (j < valid) {
                                            float v = a_u * __uint_as_float(r[j]);
                                            if (b_u != 0.0f) v = __fmaf_rn(b_u, __half2float(*c16), v);
                                            *dst16 = __float2half_rn(v);
                                        }
                                        dst16 += pitch;
                                        c16 += pitch;
                                    }
                                }
                            } else if (b_u == 0.0f) {
    #pragma unroll
                                for (int j = 0; j < 32; ++j) {
                                    if (j < 16 || wide) {
                                        if (j < valid) *dst = a_u * __uint_as_float(r[j]);
                                        dst += pitch;
                                    }
                                }
                            } else {
    #pragma unroll
                                for (int j = 0; j < 32; ++j) {
                                    if (j < 16 || wide) {
                                        if (j < valid) *dst = __fmaf_rn(b_u, __ldg(csrc), __fmul_rn(a_u, __uint_as_float(r[j])));
                                        dst += pitch;
                                        csrc += pitch;
                                    }
                                }
                            }
                        }
                    } else if (out_half) {
                        // fp16 C and D: four values per 8-byte store
                        if (row_ok) {
                            uint2 *dst = reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(gD) + row_off + c0);
                            const uint2 *csrc = reinterpret_cast<const uint2 *>(reinterpret_cast<const __half *>(gC) + row_off + c0);
    #pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                if (j < nvec && w.n0 + c0 + 4 * j < c.N) {
                                    float4 v;
                                    v.x = a_u * __uint_as_float(r[4 * j + 0]);
                                    v.y = a_u * __uint_as_float(r[4 * j + 1]);
                                    v.z = a_u * __uint_as_float(r[4 * j + 2]);
                                    v.w = a_u * __uint_as_float(r[4 * j + 3]);
                                    if (b_u != 0.0f) {
                                        const uint2 cv = __ldg(csrc + j);
                                        const float2 c01 = __half22float2(*reinterpret_cast<const __half2 *>(&cv.x));
                                        const float2 c23 = __half22float2(*reinterpret_cast<const __half2 *>(&cv.y));
                                        v.x = __fmaf_rn(b_u, c01.x, v.x);
                                        v.y = __fmaf_rn(b_u, c01.y, v.y);
                                        v.z = __fmaf_rn(b_u, c23.x, v.z);
                                        v.w = __fmaf_rn(b_u, c23.y, v.w);
                                    }
                                    const __half2 h01 = __floats2half2_rn(v.x, v.y), h23 = __floats2half2_rn(v.z, v.w);
                                    uint2 o;
                                    o.x = *reinterpret_cast<const uint32_t *>(&h01);
                                    o.y = *reinterpret_cast<const uint32_t *>(&h23);
                                    dst[j] = o;
                                }
                            }
                        }
                    } else if (c.epi_mode == 0 || !wide) {
                        if (row_ok) {
                            float4 *dst = reinterpret_cast<float4 *>(out + row_off + c0);
                            const float4 *csrc = reinterpret_cast<const float4 *>(gC + row_off + c0);
    #pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                if (j < nvec && w.n0 + c0 + 4 * j < c.N) {
                                    float4 v;
                                    v.x = a_u * __uint_as_float(r[4 * j + 0]);
                                    v.y = a_u * __uint_as_float(r[4 * j + 1]);
                                    v.z = a_u * __uint_as_float(r[4 * j + 2]);
                                    v.w = a_u * __uint_as_float(r[4 * j + 3]);
                                    if (b_u != 0.0f) {
                                        const float4 cv = __ldg(csrc + j);
                                        v.x = __fmaf_rn(b_u, cv.x, v.x);
                                        v.y = __fmaf_rn(b_u, cv.y, v.y);
                                        v.z = __fmaf_rn(b_u, cv.z, v.z);
                                        v.w = __fmaf_rn(b_u, cv.w, v.w);
                                    }
                                    dst[j] = v;
                                }
                            }
                        }
                    } else {
                        // registers -> 128-byte-swizzled shared memory -> one TMA store of 32 x 32 fp32 (the boxes the common
                        // drain above does not take: ragged tile columns, the finishing CTA of a cut tile)
                        const uint32_t buf = epi_buf + (store_idx & two_bufs) * 4096u;
                        if (lane == 0) {   // the box stored two steps ago (one step ago with a single box) has been read
                            if (two_bufs) tma_store_wait_read<1>();
                            else tma_store_wait_read<0>();
                        }
                        __syncwarp();
                        const float4 *csrc = reinterpret_cast<const float4 *>(gC + row_off + c0);
    #pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float4 v;
                            v.x = a_u * __uint_as_float(r[4 * j + 0]);
                            v.y = a_u * __uint_as_float(r[4 * j + 1]);
                            v.z = a_u * __uint_as_float(r[4 * j + 2]);
                            v.w = a_u * __uint_as_float(r[4 * j + 3]);
                            if (b_u != 0.0f && row_ok && w.n0 + c0 + 4 * j < c.N) {
                                const float4 cv = __ldg(csrc + j);
                                v.x = __fmaf_rn(b_u, cv.x, v.x);
                                v.y = __fmaf_rn(b_u, cv.y, v.y);
                                v.z = __fmaf_rn(b_u, cv.z, v.z);
                                v.w = __fmaf_rn(b_u, cv.w, v.w);
                            }
                            const uint32_t addr = buf + static_cast<uint32_t>(lane) * 128u + static_cast<uint32_t>((j ^ (lane & 7)) * 16);
                            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z),
                                         "f"(v.w)
                                         : "memory");
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d_hint(&g.map_d, buf, w.n0 + c0, row - lane, d_policy);   // the first of this warp's 32 rows (128-row atoms: row = ... + lane)
                            tma_store_commit();
                        }
                        ++store_idx;
                    }
                }
                if (atom_release && mh == 0) upper_atom_drained();
            }   // atoms
            if (w.kind == 2) {
                // this warp's part of the partial is complete: make it visible, then say so
                __threadfence();
                __syncwarp();
                if (lane == 0 && !(dbg & 16)) {
                    __threadfence();
                    *(tail_flags + tail_slot * 8 + e) = tail_epoch;
                }
            }
            // accumulator slot drained: hand it back to the MMA thread
            if (e == 0 && lane == 0) B200_TL(23);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if constexpr (CG == 2) mbar_arrive_cluster(tmem_empty_leader + 8u * (atom_release ? 1u : acc));
                else mbar_arrive(tmem_empty0 + 8u * (atom_release ? 1u : acc));
            }
        }
        if (e == 0 && lane == 0) B200_TL(24);
        if (c.epi_mode && lane == 0) tma_store_wait<0>();
        if (push_world > 0) __threadfence_system();  // this thread's peer stores are ordered before the flag below
        __syncwarp();
        if (prof && e == 0 && lane == 0) {
            prof[10] = t_tfull;
            prof[11] = clock64() - t_begin;
            prof[12] = tl;
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (clustered) {
        // no CTA leaves while a peer may still arrive on its barriers or read its shared memory
        cluster_arrive();
        cluster_wait();
    }
    if (push_world > 0 && tid == 0) {
        // Count finished CTAs; the last one tells every owner that this rank's slots are complete.
        // Every CTA counts, aborted or not, and the last one always zeroes the counter, so a launch
        // that timed out leaves it ready for the next one; the flags are raised only when no wait of
        // this launch expired (a CTA records its timeout in the status word before it counts).
        __threadfence();
        const unsigned int done = atomicAdd(g.push_done, 1u);
        if (done == gridDim.x - 1) {
            __threadfence_system();
            if (*reinterpret_cast<volatile int *>(&g_device_status[0]) == 0)
                for (int o = 0; o < push_world; ++o) *reinterpret_cast<volatile int *>(g.push_flag[o] + push_rank) = g.push_epoch;
            __threadfence_system();
            *g.push_done = 0u;
        }
    }
    if (warp == mma_warp) {
        if (*abort_flag) {
            // give copies and MMAs still in flight a bounded time to land before the memory goes
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {
            }
        }
        tc_fence_after_sync();
        tmem_dealloc<CG>(tmem_base, static_cast<uint32_t>(tmem_cols));
    }
    if (PROF && prof && tid == 0) prof[15] = static_cast<long long>(global_timer_ns());  // roles and teardown done
}

// D = alpha * sum_s partial[s] + beta * C, the second step of split-K. Slices are summed in
// ascending order, so the result does not depend on scheduling.
__global__ void splitk_reduce_kernel(const float4 *__restrict__ partial, const float4 *__restrict__ C,
                                     float4 *__restrict__ D, float alpha, float beta, long long n4, int split_k) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 s = partial[i];
        for (int k = 1; k < split_k; ++k) {
            const float4 v = partial[static_cast<long long>(k) * n4 + i];
            s.x += v.x;
            s.y += v.y;
            s.z += v.z;
            s.w += v.w;
        }
        float4 o;
        o.x = alpha * s.x;
        o.y = alpha * s.y;
        o.z = alpha * s.z;
        o.w = alpha * s.w;
        if (beta != 0.0f) {
            const float4 c = C[i];
            o.x = __fmaf_rn(beta, c.x, o.x);
            o.y = __fmaf_rn(beta, c.y, o.y);
            o.z = __fmaf_rn(beta, c.z, o.z);
            o.w = __fmaf_rn(beta, c.w, o.w);
        }
        D[i] = o;
    }
}

// Owner side of the fused split-K exchange. Block-wide bounded wait on the source ranks' flags
// (written by peers over NVLink), then an ordered sum of the slots. Slots are read with .cg loads:
// they were written by other GPUs, L1 is not coherent with those writes.
__global__ void push_reduce_kernel(const float4 *slots, const int *flags, int world, int epoch, const float4 *__restrict__ C,
                                   float4 *__restrict__ D, float alpha, float beta, long long n4, long long budget) {
    __shared__ int ok_flag;
    if (threadIdx.x == 0) {
        const long long t0 = clock64();
        int ok = 1;
        for (int s = 0; s < world && ok; ++s) {
            // Epochs only grow, so a flag past `epoch` also means "epoch `epoch` has arrived": the source
            // may already have pushed its next step (into the other slot area) before this owner looked.
            while (static_cast<int>(*reinterpret_cast<const volatile int *>(flags + s) - epoch) < 0) {
                __nanosleep(200);
                if (clock64() - t0 > budget) {
                    ok = 0;
                    if (atomicCAS(&g_device_status[0], 0, B200_DEVICE_TIMEOUT) == 0) {
                        g_device_status[1] = static_cast<int>(blockIdx.x);
                        g_device_status[2] = 700 + s;
                        g_device_status[3] = epoch;
                    }
                    break;
                }
            }
        }
        __threadfence_system();
        ok_flag = ok;
    }
    __syncthreads();
    if (!ok_flag) return;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 s = __ldcg(slots + i);
        for (int k = 1; k < world; ++k) {
            const float4 v = __ldcg(slots + static_cast<long long>(k) * n4 + i);
            s.x += v.x;
            s.y += v.y;
            s.z += v.z;
            s.w += v.w;
        }
        float4 o;
        o.x = alpha * s.x;
        o.y = alpha * s.y;
        o.z = alpha * s.z;
        o.w = alpha * s.w;
        if (beta != 0.0f) {
            const float4 c = C[i];
            o.x = __fmaf_rn(beta, c.x, o.x);
            o.y = __fmaf_rn(beta, c.y, o.y);
            o.z = __fmaf_rn(beta, c.z, o.z);
            o.w = __fmaf_rn(beta, c.w, o.w);
        }
        D[i] = o;
    }
}

// Split-K inside the GPU combined with the exchange across GPUs: sums this rank's K slices
// (ascending order) and stores each row of the sum into the slot area of the GPU that owns the
// row (coalesced 128-bit peer stores over NVLink); the last block raises this rank's flags.
struct PushDest {
    float *slot[8];
    int *flag[8];
    unsigned int *done;
    int world, rank, rows, epoch;
};

__global__ void splitk_reduce_push_kernel(const float4 *__restrict__ partial, long long n4, int split_k, int n_cols4,
                                          const __grid_constant__ PushDest d) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 s = partial[i];
        for (int k = 1; k < split_k; ++k) {
            const float4 v = partial[static_cast<long long>(k) * n4 + i];
            s.x += v.x;
            s.y += v.y;
            s.z += v.z;
            s.w += v.w;
        }
        const long long row = i / n_cols4;
        const int owner = static_cast<int>(row / d.rows);
        const long long dst = (static_cast<long long>(d.rank) * d.rows + (row - static_cast<long long>(owner) * d.rows)) * n_cols4 + i % n_cols4;
        reinterpret_cast<float4 *>(d.slot[owner])[dst] = s;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int done = atomicAdd(d.done, 1u);
        if (done == gridDim.x - 1) {
            __threadfence_system();
            for (int o = 0; o < d.world; ++o) *reinterpret_cast<volatile int *>(d.flag[o] + d.rank) = d.epoch;
            __threadfence_system();
            *d.done = 0u;
        }
    }
}

int launch_splitk_reduce_push(const float *partial, int64_t m, int64_t n, int split_k, float *const *slots, int *const *flags,
                              unsigned int *done, int world, int rank, int epoch, cudaStream_t stream) {
    PushDest d = {};
    for (int o = 0; o < world; ++o) {
        d.slot[o] = slots[o];
        d.flag[o] = flags[o];
    }
    d.done = done;
    d.world = world;
    d.rank = rank;
    d.rows = static_cast<int>(m / world);
    d.epoch = epoch;
    const long long n4 = m * n / 4;
    int blocks = static_cast<int>((n4 + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    splitk_reduce_push_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float4 *>(partial), n4, split_k,
                                                          static_cast<int>(n / 4), d);
    return static_cast<int>(cudaGetLastError());
}

// Flags between the GPUs of a box (plain ints in peer-mapped device memory): one thread writes a flag after
// everything before it in the stream has completed; one thread waits, bounded, until a flag has reached an epoch
// (epochs only grow). A wait that runs out leaves a DEVICE_TIMEOUT record {block 0, wait id, epoch}.
__global__ void flag_set_kernel(int *flag, int epoch) {
    __threadfence_system();
    *reinterpret_cast<volatile int *>(flag) = epoch;
    __threadfence_system();
}

__global__ void flag_wait_kernel(const int *flag, int epoch, long long budget, int wait_id) {
    const long long t0 = clock64();
    while (static_cast<int>(*reinterpret_cast<const volatile int *>(flag) - epoch) < 0) {
        __nanosleep(200);
        if (clock64() - t0 > budget) {
            if (atomicCAS(&g_device_status[0], 0, B200_DEVICE_TIMEOUT) == 0) {
                g_device_status[1] = 0;
                g_device_status[2] = wait_id;
                g_device_status[3] = epoch;
            }
            break;
        }
    }
    __threadfence_system();
}

int launch_flag_set(int *flag, int epoch, cudaStream_t stream) {
    flag_set_kernel<<<1, 1, 0, stream>>>(flag, epoch);
    return static_cast<int>(cudaGetLastError());
}

int launch_flag_wait(const int *flag, int epoch, long long budget_cycles, int wait_id, cudaStream_t stream) {
    flag_wait_kernel<<<1, 1, 0, stream>>>(flag, epoch, budget_cycles, wait_id);
    return static_cast<int>(cudaGetLastError());
}

int launch_push_reduce(const float *slots, const int *flags, int world, int epoch, const float *C, float *D, float alpha,
                       float beta, int64_t rows, int64_t n, long long budget_cycles, cudaStream_t stream) {
    const long long n4 = rows * n / 4;
    int blocks = static_cast<int>((n4 + 255) / 256);
    if (blocks > 148 * 4) blocks = 148 * 4;
    if (blocks < 1) blocks = 1;
    push_reduce_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float4 *>(slots), flags, world, epoch,
                                                   reinterpret_cast<const float4 *>(C), reinterpret_cast<float4 *>(D), alpha,
                                                   beta, n4, budget_cycles);
    return static_cast<int>(cudaGetLastError());
}

namespace {
typedef void (*KernelFn)(const GemmArgs);

KernelFn pick_kernel(int cta_group, bool simple, bool prof) {
    if (cta_group == 2) {
        if (simple) return prof ? gemm_sm100_kernel<2, true, true> : gemm_sm100_kernel<2, true, false>;
        return prof ? gemm_sm100_kernel<2, false, true> : gemm_sm100_kernel<2, false, false>;
    }
    if (simple) return prof ? gemm_sm100_kernel<1, true, true> : gemm_sm100_kernel<1, true, false>;
    return prof ? gemm_sm100_kernel<1, false, true> : gemm_sm100_kernel<1, false, false>;
}

// How many clusters of the launch's size the current device holds at once (it depends on how the
// SMs are grouped), asked once per {device, kernel instance, cluster size, shared-memory size}
// and remembered; -1 = the runtime could not say. Callers on different host threads share the
// table, hence the lock.
int max_active_clusters(KernelFn fn, const cudaLaunchConfig_t &cfg, int cluster) {
    struct Entry {
        int dev;
        KernelFn fn;
        int cluster;
        size_t smem;
        int value;
    };
    static std::mutex mu;
    static std::vector<Entry> table;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    for (const Entry &e : table)
        if (e.dev == dev && e.fn == fn && e.cluster == cluster && e.smem == cfg.dynamicSmemBytes) return e.value;
    int n = 0;
    const int value = (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) == cudaSuccess && n > 0) ? n : -1;
    cudaGetLastError();
    table.push_back({dev, fn, cluster, cfg.dynamicSmemBytes, value});
    return value;
}
}  // namespace

int profile_slots() { return kProfSlots; }

int prepare_kernels() {
    for (int cg = 1; cg <= 2; ++cg)
        for (int simple = 0; simple < 2; ++simple)
            for (int prof = 0; prof < 2; ++prof) {
                const cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void *>(pick_kernel(cg, simple != 0, prof != 0)),
                                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
                if (e != cudaSuccess) return static_cast<int>(e);
            }
    return 0;
}

int launch_gemm(const Plan &p, const GemmArgs &args, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    int grid = p.grid;
    if (p.cluster_reduce) {
        // whole clusters only, and no more of them than there are tiles
        const int per_tile = p.split_k * p.cta_group;
        grid -= grid % per_tile;
        if (grid > args.num_tiles * per_tile) grid = args.num_tiles * per_tile;
        if (grid < per_tile) grid = per_tile;
    }
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(static_cast<unsigned>(p.threads), 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(p.smem_bytes);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = nullptr;
    cfg.numAttrs = 0;
    const int cluster = p.cta_group * (p.cluster_reduce ? p.split_k : 1);
    if (cluster > 1) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    const bool simple = (p.a_bars == 1 && p.b_bars == 1 && p.a_boxes == 1 && p.b_priv == 0 && p.b_res_chunks == 1);
    if (args.overlap_launch) {
        attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs += 1;
    }
    const KernelFn fn = pick_kernel(p.cta_group, simple, args.prof != nullptr);
    if (p.cluster_reduce) {
        // A persistent grid wants every cluster resident at once: ask how many clusters of this
        // size the device holds (it depends on how the SMs are grouped) and cap the grid there.
        const int mc = max_active_clusters(fn, cfg, cluster);
        if (mc > 0 && grid > mc * cluster) cfg.gridDim = dim3(static_cast<unsigned>(mc * cluster), 1, 1);
    }
    const cudaError_t e = cudaLaunchKernelEx(&cfg, fn, args);
    return static_cast<int>(e);
}

int launch_splitk_reduce(const float *partial, const float *C, float *D, float alpha, float beta, int64_t mn,
                         int split_k, cudaStream_t stream) {
    const long long n4 = mn / 4;
    int blocks = static_cast<int>((n4 + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float4 *>(partial),
                                                     reinterpret_cast<const float4 *>(C), reinterpret_cast<float4 *>(D),
                                                     alpha, beta, n4, split_k);
    return static_cast<int>(cudaGetLastError());
}

int read_device_status(int out[4], cudaStream_t stream) {
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return static_cast<int>(e);
    int host[4] = {0, 0, 0, 0};
    e = cudaMemcpyFromSymbol(host, g_device_status, sizeof(host));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (host[0] != 0) {
        const int zero[4] = {0, 0, 0, 0};
        e = cudaMemcpyToSymbol(g_device_status, zero, sizeof(zero));
        if (e != cudaSuccess) return static_cast<int>(e);
        // a launch that timed out may have left tail-split flags raised that nobody consumed
        void *flags = nullptr;
        e = cudaGetSymbolAddress(&flags, g_tail_flags);
        if (e == cudaSuccess) e = cudaMemset(flags, 0, sizeof(unsigned int) * kTailSets * kTailMaxSlots * 8);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    for (int i = 0; i < 4; ++i) out[i] = host[i];
    return 0;
}

}  // namespace b200
