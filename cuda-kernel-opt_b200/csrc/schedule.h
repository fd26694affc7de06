// The work schedule of the persistent GEMM kernel: which tiles and K ranges a CTA (or CTA pair) processes,
// in which order. Plain integer arithmetic shared by the kernel (every role of a CTA walks the same sequence)
// and by the host (b200_gemm_schedule lists it for tests and tuners), so it compiles for both.
//
// Successor of the reference's persistent tile loop and its tile order (matmul_shmem_tc_async.cu:251-255,
// get_tile_offset_cd in matmul_shmem_tc_async_opt_port_0.cu:201-210).
#pragma once

#include <cstdint>

#ifdef __CUDACC__
#define B200_HD __host__ __device__ __forceinline__
#else
#define B200_HD inline
#endif

namespace b200 {

B200_HD int sched_min(int a, int b) { return a < b ? a : b; }

struct Unit {
    int m0, n0, slice, seg_begin, seg_end;
    // tail split: 0 = a whole tile, 1 = the last K slice of a cut tile (this CTA finishes the tile: adds the other
    // slices' partials and writes D), 2 = an earlier K slice (raw accumulator to slot `slot` of the workspace)
    int kind;
    int slot;      // kind 2: this unit's partial slot; kind 1: the slot of the tile's slice 0 (slice i: slot + i * tiles)
};

// Launch constants the role loops need, copied once from the kernel parameter into registers.
// The parameter is __grid_constant__ and its address escapes (tensor maps), so reading a field
// after an asm statement with a memory clobber is a fresh load through the parameter window;
// those loads sat on the critical path of the single-thread producer and MMA loops.
struct Cfg {
    int num_units, num_tiles, tiles_m, tiles_n, tile_group_m, tile_m, tile_n, num_segs, split_k;
    int tail_tiles, tail_slices;  // tail split: the first tail_tiles tiles are cut into tail_slices K slices each
    int kblocks, stages, stage_bytes, a_stage_bytes, cta_rows_a;
    int a_box_rows, a_boxes, a_priv, a_bars, chunk_n, b_priv, b_res_chunks, b_bars;
    int acc_cols, mma_m, epi_mode, epi_warps, M, N;
    int cl_split, cl_rank;  // cluster reduce: K slices per tile (= cluster size) and this CTA's slice
    int cl_seg_begin, cl_seg_end;
    uint32_t idesc_chunk, idesc_res;
    long long budget;
};

// Tile index -> tile origin. Tiles follow the reference's grouped order (get_tile_offset_cd,
// port_0.cu:201-210): tile_group_m tile rows are walked column-major inside a group so concurrently
// running CTAs share B^T column panels in L2; the last group may be short.
B200_HD void tile_origin(const Cfg &c, int t, Unit &w) {
    if (c.tiles_m == 1) {
        // one row of tiles (the skinny shapes): the grouped order is the plain column order
        w.m0 = 0;
        w.n0 = t * c.tile_n;
        return;
    }
    if (c.tiles_n == 1) {
        // one column of tiles (the skinny shapes with swapped roles): the grouped order is the plain row order
        w.m0 = t * c.tile_m;
        w.n0 = 0;
        return;
    }
    const int group_tile_count = c.tile_group_m * c.tiles_n;
    const int group_first_row = (t / group_tile_count) * c.tile_group_m;
    const int group_rows = sched_min(c.tiles_m - group_first_row, c.tile_group_m);
    const int in_group = t % group_tile_count;
    w.m0 = (group_first_row + in_group % group_rows) * c.tile_m;
    w.n0 = (in_group / group_rows) * c.tile_n;
}

// Work unit -> tile and K slice (every schedule but the tail split).
B200_HD Unit decode_unit(const Cfg &c, int u) {
    // The roles that call this are single dependent instruction chains, where an integer
    // division costs on the order of a hundred cycles: the common cases avoid them.
    Unit w;
    int t;
    w.kind = 0;
    w.slot = 0;
    if (c.cl_split > 1) {
        t = u;
        w.slice = c.cl_rank;
        w.seg_begin = c.cl_seg_begin;   // the same K slice for every tile of this CTA
        w.seg_end = c.cl_seg_end;
    } else if (c.split_k == 1) {
        t = u;
        w.slice = 0;
        w.seg_begin = 0;
        w.seg_end = c.num_segs;
    } else {
        t = u % c.num_tiles;
        w.slice = u / c.num_tiles;
        // slice <= 64 and num_segs < 2^24: the products fit 32 bits
        w.seg_begin = static_cast<int>(static_cast<unsigned>(w.slice) * static_cast<unsigned>(c.num_segs) / static_cast<unsigned>(c.split_k));
        w.seg_end = static_cast<int>(static_cast<unsigned>(w.slice + 1) * static_cast<unsigned>(c.num_segs) / static_cast<unsigned>(c.split_k));
    }
    tile_origin(c, t, w);
    return w;
}

// The sequence of work units of one CTA group; every role of the CTA walks the same sequence.
// Plain schedules: units group, group + num_groups, ... Tail split: first this group's K-slice units of the
// cut tiles (unit p = slice * tail_tiles + tile, dealt out in rounds: p = group, group + num_groups, ...), then
// whole tiles of the rest, one per wave.
struct Walk {
    int u;         // plain schedules: next unit; tail split: next slice unit
    int dp_tile;   // tail split: next whole tile
};

B200_HD void walk_init(const Cfg &c, Walk &k, int group) {
    k.u = group;
    k.dp_tile = c.tail_tiles + group;
}

B200_HD bool walk_next(const Cfg &c, Walk &k, int num_groups, Unit &w) {
    if (c.tail_tiles == 0) {
        if (k.u >= c.num_units) return false;
        w = decode_unit(c, k.u);
        k.u += num_groups;
        return true;
    }
    int t;
    if (k.u < c.tail_tiles * c.tail_slices) {
        const int sl = k.u / c.tail_tiles;
        t = k.u - sl * c.tail_tiles;
        w.slice = sl;
        w.seg_begin = static_cast<int>(static_cast<unsigned>(sl) * static_cast<unsigned>(c.num_segs) / static_cast<unsigned>(c.tail_slices));
        w.seg_end = static_cast<int>(static_cast<unsigned>(sl + 1) * static_cast<unsigned>(c.num_segs) / static_cast<unsigned>(c.tail_slices));
        w.kind = (sl == c.tail_slices - 1) ? 1 : 2;
        w.slot = (w.kind == 2) ? k.u : t;
        k.u += num_groups;
    } else if (k.dp_tile < c.num_tiles) {
        t = k.dp_tile;
        k.dp_tile += num_groups;
        w.slice = 0;
        w.seg_begin = 0;
        w.seg_end = c.num_segs;
        w.kind = 0;
        w.slot = 0;
    } else {
        return false;
    }
    tile_origin(c, t, w);
    return true;
}

}  // namespace b200
