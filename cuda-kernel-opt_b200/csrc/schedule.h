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
    // stream-K: 0 = a whole tile (or a tile that ends up whole in this CTA), 1 = the first K iterations of a
    // tile that other CTAs continue (this CTA finishes it: adds their partials and writes D), 2 = a later
    // part of a tile another CTA finishes (raw accumulator to this CTA's slot of the workspace)
    int kind;
    int tile_end;  // kind 1: the stream-K iteration index at which this tile ends (finds the peers)
};


// Launch constants the role loops need, copied once from the kernel parameter into registers.
// The parameter is __grid_constant__ and its address escapes (tensor maps), so reading a field
// after an asm statement with a memory clobber is a fresh load through the parameter window;
// those loads sat on the critical path of the single-thread producer and MMA loops.
struct Cfg {
    int num_units, num_tiles, tiles_m, tiles_n, tile_group_m, tile_m, tile_n, num_segs, split_k;
    int sk_tiles, sk_lo, sk_hi;  // stream-K region (tiles) and this CTA group's range of its K iterations
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
    const int group_tile_count = c.tile_group_m * c.tiles_n;
    const int group_first_row = (t / group_tile_count) * c.tile_group_m;
    const int group_rows = sched_min(c.tiles_m - group_first_row, c.tile_group_m);
    const int in_group = t % group_tile_count;
    w.m0 = (group_first_row + in_group % group_rows) * c.tile_m;
    w.n0 = (in_group / group_rows) * c.tile_n;
}

// Work unit -> tile and K slice (every schedule but stream-K).
B200_HD Unit decode_unit(const Cfg &c, int u) {
    // The roles that call this are single dependent instruction chains, where an integer
    // division costs on the order of a hundred cycles: the common cases avoid them.
    Unit w;
    int t;
    w.kind = 0;
    w.tile_end = 0;
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

// First stream-K iteration of CTA group g: the region's iterations dealt out in num_groups equal ranges.
B200_HD int sk_range_begin(int g, int sk_tiles, int num_segs, int num_groups) {
    return static_cast<int>(static_cast<long long>(g) * sk_tiles * num_segs / num_groups);
}

// The sequence of work units of one CTA group; every role of the CTA walks the same sequence.
// Plain schedules: units group, group + num_groups, ... Stream-K: first the pieces of this group's
// range of the region's K iterations (the end of a tile, whole tiles, the beginning of a tile), then
// whole tiles of the rest, one per wave.
struct Walk {
    int u;                           // plain schedules: next unit
    int sk_pos, sk_tile, sk_first;   // stream-K: next iteration; the tile it belongs to; that tile's first iteration
    int dp_tile;                     // next whole tile after the region
};

B200_HD void walk_init(const Cfg &c, Walk &k, int group) {
    k.u = group;
    k.sk_pos = c.sk_lo;
    k.sk_tile = c.sk_tiles > 0 ? c.sk_lo / c.num_segs : 0;
    k.sk_first = k.sk_tile * c.num_segs;
    k.dp_tile = c.sk_tiles + group;
}

B200_HD bool walk_next(const Cfg &c, Walk &k, int num_groups, Unit &w) {
    if (c.sk_tiles == 0) {
        if (k.u >= c.num_units) return false;
        w = decode_unit(c, k.u);
        k.u += num_groups;
        return true;
    }
    int t;
    if (k.sk_pos < c.sk_hi) {
        t = k.sk_tile;
        const int tile_end = k.sk_first + c.num_segs;
        const int end = sched_min(c.sk_hi, tile_end);
        w.seg_begin = k.sk_pos - k.sk_first;
        w.seg_end = end - k.sk_first;
        w.kind = w.seg_begin > 0 ? 2 : (end < tile_end ? 1 : 0);
        w.tile_end = tile_end;
        k.sk_pos = end;
        k.sk_tile += 1;
        k.sk_first = tile_end;
    } else if (k.dp_tile < c.num_tiles) {
        t = k.dp_tile;
        k.dp_tile += num_groups;
        w.seg_begin = 0;
        w.seg_end = c.num_segs;
        w.kind = 0;
        w.tile_end = 0;
    } else {
        return false;
    }
    w.slice = 0;
    tile_origin(c, t, w);
    return true;
}

}  // namespace b200
