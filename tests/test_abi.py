"""CPU: the C-ABI library loads, exports every symbol the headers declare, and its host-only
planning (the reference launcher's asserts and shared-memory filter as return codes) behaves.
No compute entry point is called here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200_gemm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    lib = ctypes.CDLL(pkg.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/b200_gemm.h but not exported"
    assert sorted(pkg.EXPORTS) == names, "package binding list and header disagree"


def test_cpp_launcher_header_compiles(tmp_path):
    """include/b200_matmul.h: the four reference argument lists (15/16/18/20) resolve."""
    src = tmp_path / "t.cpp"
    src.write_text('''
#include "b200_matmul.h"
using namespace b200_matmul;
int f(const half* A, const half* B, const float* C, float* D, const __nv_bfloat16* X) {
  int s = gemm_shmem_tc_async<half, float>(A, B, C, D, 1.f, 1.f, 128, 128, 128, 128, 64, 2, 1, 4, 148);
  s += gemm_shmem_tc_async_opt_port<half, float>(A, B, C, D, 1.f, 1.f, 128, 128, 128, 128, 64, 2, 2, 1, 4, 148);
  s += gemm_shmem_tc_async_opt_port<half, float>(A, B, C, D, 1.f, 1.f, 128, 128, 128, 128, 64, 64, 64, 2, 2, 2, 4, 148);
  s += gemm_shmem_tc_async_opt_port<half, float>(A, B, C, D, 1.f, 1.f, 128, 128, 128, 128, 64, 1, 1, 64, 64, 2, 2, 2, 4, 148);
  s += gemm_shmem_tc_async_opt_port<__nv_bfloat16, float>(X, X, C, D, 1.f, 0.f, 128, 128, 128, 128, 64, 2, 2, 1, 4, 148);
  return s + get_shmem_req(128, 64, 1, 1, 64, 64, 3, 4) + get_num_acc(128, 4) + get_warp_tile_rows(64, 8);
}
''')
    import subprocess
    r = subprocess.run(["/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++", "-std=c++17", "-fsyntax-only",
                        "-I", os.path.join(ROOT, "include"), "-I", "/usr/local/cuda/include", str(src)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def P(pkg, **ov):
    base = dict(tile_m=128, tile_n=128, segment_dim_k=64, bar_steps_a=0, bar_steps_b=0, bar_step_rows_a=128,
                bar_step_rows_b=128, tile_group_m=1, num_stages=2, num_producer_warps=2, num_consumer_warps=4,
                num_sms=148, cta_group=1, split_k=1, epilogue=0)
    base.update(ov)
    p = pkg.Params()
    for k, v in base.items():
        setattr(p, k, v)
    return p


def test_reference_parameter_domain(pkg):
    """The asserts of the reference launchers (matmul_shmem_tc_async.cu:511-517,
    matmul_shmem_tc_async_opt_port_2.cu:1112-1123) as statuses."""
    ok = lambda **ov: pkg.validate(ov.pop("M", 1024), ov.pop("N", 1024), ov.pop("K", 1024), pkg.F16, P(pkg, **ov))
    assert ok() == pkg.OK
    for tile in (64, 128):
        assert ok(tile_m=tile, tile_n=tile, bar_step_rows_a=tile, bar_step_rows_b=tile) == pkg.OK
    assert ok(tile_m=96, bar_step_rows_a=96) == pkg.INVALID_CONFIG            # tile_dim in {64, 128}
    assert ok(segment_dim_k=32) == pkg.INVALID_CONFIG                          # seg_k >= 64, % 64
    assert ok(segment_dim_k=96) == pkg.INVALID_CONFIG
    assert ok(num_stages=0) == pkg.INVALID_CONFIG                              # num_stages > 0
    assert ok(num_stages=17) == pkg.INVALID_CONFIG                             # NUM_STAGES_MAX = 16
    assert ok(tile_group_m=0) == pkg.INVALID_CONFIG                            # tile_group_m > 0
    for p_ in (1, 2, 4, 8):
        assert ok(num_producer_warps=p_) == pkg.OK
    assert ok(num_producer_warps=3) == pkg.INVALID_CONFIG
    assert ok(num_consumer_warps=8) == pkg.OK
    assert ok(num_consumer_warps=6) == pkg.INVALID_CONFIG
    assert ok(N=1002) == pkg.INVALID_SHAPE                                     # rows of D must be 16-byte multiples
    assert ok(K=1004) == pkg.INVALID_SHAPE                                     # rows of A, B^T must be 16-byte multiples
    assert ok(N=1000) == pkg.OK and ok(K=1000) == pkg.OK                       # ragged tiles are an extension of the C ABI
    assert ok(segment_dim_k=256, K=1024, num_stages=1) == pkg.OK
    assert ok(M=0) == pkg.INVALID_SHAPE
    assert ok(M=1000) == pkg.OK                                                # (the reference-shaped C++ launchers keep its tile-multiple rule)
    assert pkg.validate(1024, 1024, 1024, 7, P(pkg)) == pkg.INVALID_CONFIG     # unknown dtype


def test_barrier_granularities(pkg):
    """bar_step_rows / bar_steps (port_2.cu:1116-1120): three granularities, bounds on the steps."""
    ok = lambda **ov: pkg.validate(1024, 1024, 1024, pkg.F16, P(pkg, **ov))
    assert ok(bar_step_rows_a=16, bar_step_rows_b=16, bar_steps_a=3, bar_steps_b=3) == pkg.OK
    assert ok(bar_step_rows_a=64, bar_step_rows_b=64, bar_steps_a=2, bar_steps_b=2) == pkg.OK
    assert ok(bar_step_rows_a=64, bar_step_rows_b=64, bar_steps_a=3, bar_steps_b=0) == pkg.INVALID_CONFIG  # > tile/step
    assert ok(bar_step_rows_a=48, bar_step_rows_b=64) == pkg.INVALID_CONFIG                                 # does not divide
    assert ok(bar_step_rows_b=24) == pkg.INVALID_CONFIG
    assert ok(bar_step_rows_a=64, bar_steps_a=-1) == pkg.INVALID_CONFIG
    # more barriers cost shared memory, as in get_shmem_req (port_2.cu:1069-1080)
    s0 = pkg.smem_bytes(pkg.F16, P(pkg, num_stages=6))
    s1 = pkg.smem_bytes(pkg.F16, P(pkg, num_stages=6, bar_step_rows_a=16, bar_step_rows_b=16, bar_steps_a=7, bar_steps_b=7))
    assert 0 < s0 < s1


def test_shared_memory_filter(pkg):
    """The harness only runs configurations that fit (port_2.cu:1229-1231); here they are refused."""
    fits = P(pkg, tile_m=128, tile_n=256, bar_step_rows_b=256, num_stages=4)
    assert pkg.smem_bytes(pkg.F16, fits) == 4 * (128 + 256) * 64 * 2 + (4 * 4 + 6) * 8 + 16 + 1024
    too_deep = P(pkg, tile_m=128, tile_n=256, bar_step_rows_b=256, num_stages=6)   # 288 KiB of stages
    assert pkg.smem_bytes(pkg.F16, too_deep) == -1
    assert pkg.validate(4096, 4096, 4096, pkg.F16, too_deep) == pkg.INVALID_CONFIG
    assert pkg.smem_bytes(pkg.F16, P(pkg, num_stages=1)) >= 116 * 1024              # one CTA per SM always
    with_tma_epilogue = P(pkg, tile_m=128, tile_n=256, bar_step_rows_b=256, num_stages=4, epilogue=1)
    assert pkg.smem_bytes(pkg.F16, with_tma_epilogue) - pkg.smem_bytes(pkg.F16, fits) == 4 * 2 * 4096


def test_b200_extensions(pkg):
    ok = lambda M=4096, N=4096, K=4096, **ov: pkg.validate(M, N, K, pkg.BF16, P(pkg, **ov))
    assert ok(tile_m=256, tile_n=256, cta_group=2, bar_step_rows_a=256, bar_step_rows_b=256, num_stages=6) == pkg.OK
    assert ok(tile_m=128, tile_n=256, cta_group=2, bar_step_rows_b=256) == pkg.INVALID_CONFIG   # a pair needs tile_m = 256
    assert ok(tile_m=256, cta_group=1, bar_step_rows_a=256) == pkg.INVALID_CONFIG
    assert ok(tile_n=224, bar_step_rows_b=224, N=28672) == pkg.OK
    assert ok(tile_n=264, bar_step_rows_b=264) == pkg.INVALID_CONFIG
    assert ok(split_k=4) == pkg.OK and ok(split_k=65) == pkg.INVALID_CONFIG
    assert ok(split_k=8, K=256) == pkg.INVALID_SHAPE                                            # fewer K segments than slices
    p = P(pkg, split_k=4)
    assert pkg.workspace_bytes(512, 256, 4096, p) == 4 * 512 * 256 * 4
    assert pkg.workspace_bytes(512, 256, 4096, P(pkg)) == 0


def test_tall_pair_tile_domain(pkg):
    """tile_m = 512 with cta_group = 2: each CTA stages 256 rows of A and issues them as two 128-row MMA atoms against one
    B^T stage; the two accumulators fill the 512 tensor-memory columns at tile_n = 256 (one slot), whole tiles and whole-stage
    A barriers only."""
    tall = dict(tile_m=512, tile_n=256, cta_group=2, bar_step_rows_a=512, bar_step_rows_b=256, tail_split=0)
    ok = lambda M=8192, N=8192, K=8192, **ov: pkg.validate(M, N, K, pkg.F16, P(pkg, **dict(tall, **ov)))
    assert ok(num_stages=4) == pkg.OK
    assert ok(num_stages=5) == pkg.INVALID_CONFIG                       # 5 x 48 KiB of stages + drain buffers do not fit
    assert ok(num_stages=3, num_consumer_warps=8) == pkg.OK
    # four stages beside eight draining warps: two staging boxes per warp do not fit, one does
    assert ok(num_stages=4, num_consumer_warps=8) == pkg.OK
    assert pkg.smem_bytes(pkg.F16, P(pkg, num_stages=4, num_consumer_warps=8, epilogue=1, **tall)) == 4 * (256 + 128) * 64 * 2 + 8 * 4096 + (4 * 4 + 6) * 8 + 16 + 1024
    assert pkg.smem_bytes(pkg.F16, P(pkg, num_stages=3, num_consumer_warps=8, epilogue=1, **tall)) == 3 * (256 + 128) * 64 * 2 + 8 * 2 * 4096 + (3 * 4 + 6) * 8 + 16 + 1024
    assert ok(num_stages=4, tile_n=128, bar_step_rows_b=128) == pkg.OK
    assert ok(num_stages=4, cta_group=1) == pkg.INVALID_CONFIG
    assert ok(num_stages=4, split_k=2) == pkg.INVALID_CONFIG
    assert ok(num_stages=4, bar_step_rows_a=128) == pkg.INVALID_CONFIG  # sub-tile barriers for A belong to the 128-row forms
    assert ok(num_stages=4, bar_step_rows_b=64, bar_steps_b=2) == pkg.INVALID_CONFIG   # ... and so do those for B^T
    assert ok(num_stages=4, bar_step_rows_b=64, bar_steps_b=0) == pkg.INVALID_CONFIG
    assert ok(num_stages=4, swap_ab=1) == pkg.INVALID_CONFIG
    assert pkg.smem_bytes(pkg.F16, P(pkg, num_stages=4, epilogue=1, **tall)) == 4 * (256 + 128) * 64 * 2 + 4 * 2 * 4096 + (4 * 4 + 6) * 8 + 16 + 1024
    # the schedule: 512-row tiles, every tile once, ragged M included
    p = P(pkg, num_stages=4, **tall)
    tiles, groups = _coverage(pkg, 1200, 768, 512, p, 8)
    assert groups == 4 and sorted(tiles) == [(m, n) for m in (0, 512, 1024) for n in (0, 256, 512)]


def test_swapped_roles_and_cluster_reduce_domain(pkg):
    """swap_ab: tile_n is the 64/128-row side, tile_m the multiple-of-16 side; cluster_reduce needs
    swap_ab, a portable cluster size and a narrow accumulator, and then no workspace."""
    ok = lambda M=16, N=4096, K=4096, **ov: pkg.validate(M, N, K, pkg.BF16, P(pkg, **ov))
    sw = dict(swap_ab=1, tile_m=16, tile_n=128, bar_step_rows_a=16, bar_step_rows_b=128)
    assert ok(**sw) == pkg.OK
    assert ok(**dict(sw, tile_m=48, bar_step_rows_a=48)) == pkg.OK
    assert ok(**dict(sw, tile_m=256, bar_step_rows_a=256, num_stages=3)) == pkg.OK
    assert ok(**dict(sw, tile_n=64, bar_step_rows_b=64)) == pkg.OK
    assert ok(**dict(sw, tile_n=256, bar_step_rows_b=256)) == pkg.INVALID_CONFIG       # the MMA's M side is 64 or 128
    assert ok(**dict(sw, tile_m=24, bar_step_rows_a=24)) == pkg.INVALID_CONFIG          # its N side a multiple of 16
    assert ok(**dict(sw, cta_group=2)) == pkg.INVALID_CONFIG                             # a pair needs tile_n = 256
    assert ok(**dict(sw, tail_split=1)) == pkg.INVALID_CONFIG
    assert ok(**dict(sw, swap_ab=2)) == pkg.INVALID_CONFIG
    assert ok(**dict(sw, overlap_launch=1)) == pkg.OK and ok(**dict(sw, overlap_launch=2)) == pkg.INVALID_CONFIG
    assert ok(**dict(sw, split_k=3)) == pkg.OK
    for s_ in (2, 4, 8):
        assert ok(**dict(sw, split_k=s_, cluster_reduce=1)) == pkg.OK
    assert ok(**dict(sw, split_k=3, cluster_reduce=1)) == pkg.INVALID_CONFIG            # cluster sizes 2, 4, 8
    assert ok(**dict(sw, split_k=1, cluster_reduce=1)) == pkg.INVALID_CONFIG
    assert ok(**dict(sw, tile_m=144, bar_step_rows_a=144, split_k=2, cluster_reduce=1)) == pkg.INVALID_CONFIG  # > 128 columns
    assert ok(tile_m=128, tile_n=128, split_k=2, cluster_reduce=1) == pkg.INVALID_CONFIG    # needs swap_ab
    assert pkg.workspace_bytes(16, 4096, 4096, P(pkg, **dict(sw, split_k=4))) == 4 * 16 * 4096 * 4
    assert pkg.workspace_bytes(16, 4096, 4096, P(pkg, **dict(sw, split_k=4, cluster_reduce=1))) == 0
    # the partial tile of a cluster reduce is staged in shared memory: 128 rows x tile_m fp32
    a = pkg.smem_bytes(pkg.BF16, P(pkg, **dict(sw, tile_m=64, bar_step_rows_a=64, num_stages=8, split_k=2)))
    b = pkg.smem_bytes(pkg.BF16, P(pkg, **dict(sw, tile_m=64, bar_step_rows_a=64, num_stages=8, split_k=2, cluster_reduce=1)))
    assert b - a == 64 * 128 * 4
    # decode-shape defaults use the swapped form, and a cluster over K when there are few tiles
    d = pkg.default_params(16, 28672, 8192, pkg.BF16)
    assert (d.swap_ab, d.tile_m, d.tile_n, d.split_k) == (1, 16, 128, 1) and pkg.validate(16, 28672, 8192, pkg.BF16, d) == pkg.OK
    d = pkg.default_params(16, 3584, 8192, pkg.BF16)
    assert (d.swap_ab, d.split_k, d.cluster_reduce) == (1, 4, 1) and pkg.validate(16, 3584, 8192, pkg.BF16, d) == pkg.OK
    d = pkg.default_params(128, 28672, 8192, pkg.BF16)                                     # swapped two-CTA pair
    assert (d.swap_ab, d.cta_group, d.tile_m, d.tile_n) == (1, 2, 128, 256) and pkg.validate(128, 28672, 8192, pkg.BF16, d) == pkg.OK
    d = pkg.default_params(128, 7168, 8192, pkg.BF16)                                      # few tiles: swapped, cluster over K
    assert (d.swap_ab, d.split_k, d.cluster_reduce) == (1, 4, 1) and pkg.validate(128, 7168, 8192, pkg.BF16, d) == pkg.OK
    d = pkg.default_params(128, 10240, 8192, pkg.BF16)                                     # in between: the plain tile
    assert d.swap_ab == 0 and pkg.validate(128, 10240, 8192, pkg.BF16, d) == pkg.OK
    # a swapped pair: 256 weight rows per tile, activation rows in multiples of 32; slices x 2 must fit a cluster of 8
    sp = dict(swap_ab=1, cta_group=2, tile_m=64, tile_n=256, bar_step_rows_a=64, bar_step_rows_b=256)
    assert ok(**sp) == pkg.OK and ok(**dict(sp, tile_m=48, bar_step_rows_a=48)) == pkg.INVALID_CONFIG
    assert ok(**dict(sp, split_k=4, cluster_reduce=1)) == pkg.OK and ok(**dict(sp, split_k=8, cluster_reduce=1)) == pkg.INVALID_CONFIG
    d = pkg.default_params(16, 28672, 8192, pkg.BF16, tile_n=64)                           # a tile override names the plain form
    assert d.swap_ab == 0 and pkg.validate(16, 28672, 8192, pkg.BF16, d) == pkg.OK


def _coverage(pkg, M, N, K, p, num_sms):
    """Walks every CTA group's schedule; returns ({(m0, n0): [(seg_begin, seg_end, kind, group), ...]}, groups)."""
    groups, _ = pkg.schedule(M, N, K, p, num_sms, 0)
    tiles = {}
    for g in range(groups):
        _, units = pkg.schedule(M, N, K, p, num_sms, g)
        for (m0, n0, sb, se, kind, sl) in units:
            tiles.setdefault((m0, n0), []).append((sb, se, kind, g))
    return tiles, groups


def test_tail_split_schedule_covers_every_k_segment_once(pkg):
    """tail_split = 1: whatever the shape, every K segment of every tile is computed by exactly one CTA group; a cut
    tile has s equal slices, the last one of kind 1 (its CTA finishes the tile), the others of kind 2; the slice
    units come first in every group's walk, slice-major in rounds; whole tiles are kind 0; and the launch gets
    shorter by what the plan promises."""
    pair = dict(tile_m=256, tile_n=256, cta_group=2, bar_step_rows_a=256, bar_step_rows_b=256, num_stages=6, tail_split=1)
    one = dict(tile_m=128, tile_n=128, tail_split=1)
    cases = [  # M, N, K, overrides, SMs, expected (cut tiles, slices) or None when nothing is gained
        (4096, 4096, 4096, pair, 148, (34, 2)),            # 256 tiles on 74 pairs: 34 left, two halves each -> 3.5 instead of 4 tile times
        (2048, 8192, 8192, pair, 148, (34, 2)),
        (1024, 8192, 8192, pair, 148, None),               # 54 left of 74: more than half a wave, one round cannot hold two slices each
        (8192, 8192, 8192, pair, 148, None),               # 62 left of 74
        (2048, 2048, 262144, pair, 148, None),             # 64 tiles on 74 pairs
        (256 * 5, 256 * 15, 2048, pair, 148, (1, 8)),      # 75 tiles: one left, eight slices (the cap)
        (128 * 3, 128 * 50, 1024, one, 148, (2, 4)),       # 150 tiles on 148: 2 left, 16 K segments -> at most 4 slices of 4
        (640, 896, 4096, one, 40, None),                   # 35 tiles on 40 CTAs
        (640, 1024, 4096, one, 30, (10, 3)),               # 40 tiles on 30 CTAs: 10 left, thirds
        (256 * 74, 256, 4096, pair, 148, None),            # a full wave
        (300, 520, 2048, dict(one, tile_n=64), 20, (7, 2)),   # 27 tiles on 20 CTAs: 7 left, halves
    ]
    for M, N, K, ov, sms, want in cases:
        p = P(pkg, **dict(ov, num_sms=sms))
        assert pkg.validate(M, N, K, pkg.F16, p) == pkg.OK
        tiles, groups = _coverage(pkg, M, N, K, p, sms)
        tm, tn, segs = p.tile_m, p.tile_n, -(-K // p.segment_dim_k)
        T = -(-M // tm) * -(-N // tn)
        assert len(tiles) == T, (M, N, K)
        cut = {k: v for k, v in tiles.items() if len(v) > 1}
        slices = {len(v) for v in cut.values()}
        assert len(slices) <= 1
        s_ = slices.pop() if slices else 1
        for (m0, n0), parts in tiles.items():
            assert m0 % tm == 0 and n0 % tn == 0 and m0 < M and n0 < N
            parts.sort()
            assert parts[0][0] == 0 and parts[-1][1] == segs, ((m0, n0), parts)
            assert all(a[1] == b[0] for a, b in zip(parts, parts[1:])), parts          # no gap, no overlap
            if len(parts) == 1:
                assert parts[0][2] == 0
            else:
                assert [k for _, _, k, _ in parts] == [2] * (s_ - 1) + [1], parts
                assert max(se - sb for sb, se, _, _ in parts) - min(se - sb for sb, se, _, _ in parts) <= 1
        longest = 0.0
        for g in range(groups):
            _, units = pkg.schedule(M, N, K, p, sms, g)
            kinds = [u[4] for u in units]
            first_whole = kinds.index(0) if 0 in kinds else len(kinds)
            assert all(k == 0 for k in kinds[first_whole:]) and first_whole <= 1, (g, kinds)   # at most one slice unit, first
            longest = max(longest, sum(u[3] - u[2] for u in units) / segs)
        if cut:
            r = len(cut)
            assert r == T % groups
            assert abs(longest - (T // groups + -(-r * s_ // groups) / s_)) < 0.06 and longest < -(-T // groups) - 0.02   # slices differ by one K segment
            assert pkg.workspace_bytes(M, N, K, p) == r * (s_ - 1) * p.cta_group * -(-tn // 32) * 16384
        else:
            assert longest == -(-T // groups)
            assert pkg.workspace_bytes(M, N, K, p) == 0
        off, _ = _coverage(pkg, M, N, K, P(pkg, **dict(ov, num_sms=sms, tail_split=0)), sms)
        assert all(len(v) == 1 and v[0][2] == 0 for v in off.values()) and set(off) == set(tiles)
        assert ((len(cut), s_) if cut else None) == want, (M, N, K, sms, len(cut), s_)
    # one K segment cannot be cut
    assert pkg.workspace_bytes(128 * 3, 128 * 50, 64, P(pkg, **one)) == 0
    with pytest.raises(ValueError):
        pkg.schedule(4096, 4096, 4096, P(pkg, **pair), 148, 74)


def test_plain_and_split_k_schedules(pkg):
    """Without the tail split: group g takes units g, g + groups, ...; split_k slices are separate units of the same tile;
    the tiles follow the reference's grouped order (tile_group_m tile rows column-major inside a group,
    matmul_shmem_tc_async_opt_port_0.cu:201-210)."""
    p = P(pkg, tile_group_m=2, num_sms=4)
    groups, u0 = pkg.schedule(512, 384, 256, p, 4, 0)
    assert groups == 4
    order = []
    for i in range(12):
        _, u = pkg.schedule(512, 384, 256, p, 4, i % 4)
        order.append(u[i // 4][:2])
    assert order == [(0, 0), (128, 0), (0, 128), (128, 128), (0, 256), (128, 256), (256, 0), (384, 0), (256, 128), (384, 128), (256, 256), (384, 256)]
    p = P(pkg, split_k=2, num_sms=8)
    tiles, groups = _coverage(pkg, 256, 256, 1024, p, 8)
    assert groups == 8 and all(sorted((sb, se) for sb, se, _, _ in v) == [(0, 8), (8, 16)] for v in tiles.values())


def test_default_params_are_valid(pkg):
    for (m, n, k) in ((1024, 1024, 1024), (4096, 4096, 4096), (8192, 8192, 8192), (16, 28672, 8192), (2048, 2048, 262144)):
        for dt in (pkg.F16, pkg.BF16):
            p = pkg.default_params(m, n, k, dt)
            assert pkg.validate(m, n, k, dt, p) == pkg.OK, (m, n, k, p.as_dict())


def test_defaults_for_large_squares_and_their_row_shards(pkg):
    """b200_gemm_default_params weighs the tall pair (512-row tiles, 256 / 224 / 192 columns) against the 256-row pair
    family by rounds of the 74 CTA pairs: 8192^3 takes 512 x 256 (seven rounds), its row shards 512 x 224 (37 tile
    columns: one, two and four whole rounds) with a fourth stage; 4096^3, a short K and a shape whose 256-wide tiles
    already fill a wave keep the 256-row pair."""
    pick = lambda m, n, k: {f: getattr(pkg.default_params(m, n, k, pkg.F16), f) for f in
                            ("tile_m", "tile_n", "cta_group", "num_stages", "num_consumer_warps", "tile_group_m", "bar_step_rows_a", "bar_step_rows_b")}
    assert pick(8192, 8192, 8192) == dict(tile_m=512, tile_n=256, cta_group=2, num_stages=3, num_consumer_warps=8, tile_group_m=8,
                                          bar_step_rows_a=512, bar_step_rows_b=256)
    for m in (1024, 2048, 4096):
        assert pick(m, 8192, 8192) == dict(tile_m=512, tile_n=224, cta_group=2, num_stages=4, num_consumer_warps=8, tile_group_m=8,
                                           bar_step_rows_a=512, bar_step_rows_b=224), m
    for shape in ((4096, 4096, 4096), (8192, 8192, 4096), (8192, 4096, 8192), (2048, 2048, 262144)):
        d = pick(*shape)
        assert (d["tile_m"], d["tile_n"], d["num_stages"], d["num_consumer_warps"]) == (256, 256, 6, 4), (shape, d)
    assert pick(512, 8192, 8192)["tile_m"] == 256 and pick(512, 8192, 8192)["tile_n"] == 224     # 2 x 37 tiles: one wave of 256 x 224 pairs
    # what a call without tunables takes when it has a C to read or writes fp16: the 256-row pair (the tall pair's exposed
    # drain only pays through the lean TMA-store path of beta = 0 and fp32 D)
    import ctypes as C
    for beta, f16_out, tile_m in ((0.0, 0, 512), (1.0, 0, 256), (0.0, 1, 256), (-0.5, 1, 256)):
        p = pkg.Params()
        assert pkg.lib().b200_gemm_default_params_for_call(8192, 8192, 8192, pkg.F16, beta, f16_out, C.byref(p)) == pkg.OK
        assert p.tile_m == tile_m and p.cta_group == 2 and pkg.validate(8192, 8192, 8192, pkg.F16, p) == pkg.OK, (beta, f16_out, p.as_dict())
    assert pkg.lib().b200_gemm_default_params_for_call(8192, 8192, 8192, pkg.F16, 0.0, 0, None) == pkg.INVALID_POINTER


def test_status_strings(pkg):
    seen = {pkg.status_string(i) for i in range(8)}
    assert len(seen) == 8 and "unknown status" not in seen
    assert pkg.status_string(99) == "unknown status"


def test_defaults_are_valid_everywhere_and_need_no_workspace(pkg):
    """b200_gemm_default_params (and its plain twin) over a grid of shapes: always a valid configuration for the
    shape, never one that needs a caller workspace (tail_split only uses one when it is
    given; K slices that must meet in a workspace are never a default), swapped forms only where the activations
    are few."""
    import itertools
    Ms = (1, 7, 16, 17, 32, 33, 64, 65, 100, 128, 129, 256, 300, 1000, 1024, 4096, 8192)
    Ns = (4, 16, 64, 100, 128, 256, 1000, 1024, 3584, 4096, 7168, 14336, 28672, 28676)
    Ks = (8, 64, 72, 512, 1000, 4096, 8192, 262144)
    for M, N, K in itertools.product(Ms, Ns, Ks):
        for dtype in (pkg.F16, pkg.BF16):
            for plain in (False, True):
                p = pkg.Params()
                fn = pkg.lib().b200_gemm_default_params_plain if plain else pkg.lib().b200_gemm_default_params
                assert fn(M, N, K, dtype, ctypes.byref(p)) == pkg.OK
                assert pkg.validate(M, N, K, dtype, p) == pkg.OK, (M, N, K, plain, p.as_dict())
                assert p.split_k == 1 or p.cluster_reduce == 1, (M, N, K, plain, p.as_dict())
                if pkg.workspace_bytes(M, N, K, p):
                    assert p.tail_split == 1 and p.swap_ab == 0
                    p.tail_split = 0
                    assert pkg.workspace_bytes(M, N, K, p) == 0, (M, N, K, plain, p.as_dict())
                assert pkg.smem_bytes(dtype, p) > 0
                if plain or M > 128:
                    assert p.swap_ab == 0
                if M <= 64 and not plain:
                    assert p.swap_ab == 1 and p.tile_m >= M
