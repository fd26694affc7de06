"""Sweep harness / autotuner for the launch tunables of one GEMM shape.

The reference explores its tunables with hard-coded nested sweeps in main() that print one line
per tuple (matmul_shmem_tc_async_opt_port_2.cu:1208-1232, :1554-1564). This is the same idea as a
tool: candidate tuples for a shape are timed round-robin (so all of them see the same clock under
the power limit), every finished candidate is appended to a JSONL file, an interrupted run resumes
where it stopped, and the best tuple can be read back.

    python cuda-kernel-opt_b200/tune.py 8192 8192 8192 --dtype f16 --out tune.jsonl

Needs a B200; there is no CPU path.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def candidates(M: int, N: int, K: int) -> list[dict]:
    """Tunable tuples worth timing for the shape: tile shape x stages x producer warps x L2 hint
    (x split-K when the tiles do not fill the GPU). Invalid ones are filtered by validate()."""
    out = []
    if M <= 128:
        # decode shapes: swapped roles (weights on the MMA's 128-row side), K over a cluster when the tiles are few
        tm = -(-M // 16) * 16
        n_tiles = -(-N // 128)
        for seg_k in (64, 128):
            per_stage = (128 + tm) * seg_k * 2
            for stages in sorted({max(2, min(10, 200000 // per_stage)), max(2, min(10, 200000 // per_stage) - 1)}):
                # every field the shape's default may set is spelled out, so a candidate is what it says
                base = dict(swap_ab=1, tile_m=tm, tile_n=128, segment_dim_k=seg_k, num_stages=stages, l2_hint=1,
                            split_k=1, cluster_reduce=0)
                out.append(base)
                if n_tiles < 148 and K >= 2048:
                    for s in (2, 4, 8):
                        out.append(dict(base, split_k=s, cluster_reduce=1))
                        out.append(dict(base, split_k=s, cluster_reduce=0))
                        if tm >= 64:      # a wide accumulator: eight draining warps halve the staging and the reduce
                            out.append(dict(base, split_k=s, cluster_reduce=1, num_consumer_warps=8))
        if M > 32:
            # the swapped two-CTA pair: 256 weight rows per tile, activation rows in multiples of 32 (each CTA stages
            # half of them); K over a cluster of 2 or 4 pairs when the pair tiles are few
            tm2 = -(-M // 32) * 32
            for seg_k in (64, 128):
                per_stage = (128 + tm2 // 2) * seg_k * 2
                for stages in sorted({max(2, min(10, 200000 // per_stage)), max(2, min(10, 200000 // per_stage) - 2)}):
                    base = dict(swap_ab=1, cta_group=2, tile_m=tm2, tile_n=256, segment_dim_k=seg_k, num_stages=stages, l2_hint=1,
                                split_k=1, cluster_reduce=0)
                    out.append(base)
                    if -(-N // 256) < 74 and K >= 2048 and tm2 <= 128:
                        for s in (2, 4):
                            out.append(dict(base, split_k=s, cluster_reduce=1))
                            out.append(dict(base, split_k=s, cluster_reduce=1, num_consumer_warps=8))
    tiles = []
    if M > 128:
        tiles += [dict(tile_m=256, tile_n=256, cta_group=2), dict(tile_m=256, tile_n=128, cta_group=2)]
    tiles += [dict(tile_m=128, tile_n=tn, cta_group=1) for tn in (256, 224, 192, 128, 64) if N % tn == 0 or tn == 128]
    if M >= 1024 and K >= 4096:
        # the tall pair: 256 rows of A per CTA as two MMA atoms; one accumulator slot, so the drain counts: eight warps
        # (256 columns, or narrower where that makes the rounds of the 74 pairs come out even; four stages beside eight
        # draining warps make them stage through one box each)
        for tn in (256, 224, 192):
            for stages, cw in ((3, 8), (4, 8), (4, 4)):
                for group in ((4, 8, 16) if tn == 256 else (8,)):
                    out.append(dict(tile_m=512, tile_n=tn, cta_group=2, bar_step_rows_a=512, bar_step_rows_b=tn, num_stages=stages,
                                    num_consumer_warps=cw, num_producer_warps=2, l2_hint=3, tile_group_m=group, k_order=1, tail_split=0))
    for t in tiles:
        per_stage = (t["tile_m"] // t["cta_group"] + t["tile_n"] // t["cta_group"]) * 128
        deepest = min(8, 200000 // per_stage)
        for stages in sorted({deepest, max(2, deepest - 2)}):
            for pw in (1, 2):
                for hint in ((0, 3) if M > 128 else (0, 1)):
                    base = dict(t, num_stages=stages, num_producer_warps=pw, l2_hint=hint)
                    out.append(base)
                    n_tiles = -(-M // t["tile_m"]) * -(-N // t["tile_n"])
                    slots = 148 // t["cta_group"]
                    if n_tiles < slots and K >= 8192:
                        for s in (2, 4, 8):
                            out.append(dict(base, split_k=s))
    return out


def key_of(params: dict) -> str:
    return json.dumps(params, sort_keys=True)


def load(path: str) -> list[dict]:
    if not os.path.exists(path):
        return []
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]


LIBRARY = {"library": "torch.matmul"}   # the vendor library timed beside the candidates (never the best: it is not this kernel)


def best(path: str, M: int, N: int, K: int, dtype: str = "f16") -> dict | None:
    rows = [r for r in load(path) if r["shape"] == [M, N, K] and r["dtype"] == dtype and r["status"] == 0 and r["params"] != LIBRARY]
    return min(rows, key=lambda r: r["ms"])["params"] if rows else None


def tune(M: int, N: int, K: int, dtype: str = "f16", out: str = "tune.jsonl", rounds: int = 12, inner: int = 3, log=print,
         with_library: bool = False):
    import torch
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    pkg = load_package()
    code = pkg.BF16 if dtype == "bf16" else pkg.F16
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float16
    done = {key_of(r["params"]) for r in load(out) if r["shape"] == [M, N, K] and r["dtype"] == dtype}
    A = torch.empty((M, K), dtype=tdt, device="cuda")
    Bt = torch.empty((N, K), dtype=tdt, device="cuda")
    pkg.fill_device(A, 1, 1)
    pkg.fill_device(Bt, 1, 2)
    D = torch.empty((M, N), dtype=torch.float32, device="cuda")
    todo = []
    for ov in candidates(M, N, K):
        if key_of(ov) in done:
            continue
        p = pkg.default_params(M, N, K, code, **ov)
        if pkg.validate(M, N, K, code, p) != pkg.OK:
            continue
        need = pkg.workspace_bytes(M, N, K, p)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        todo.append((ov, p, ws if need else None, []))
    if with_library and key_of(LIBRARY) not in done:
        todo.append((LIBRARY, None, None, []))      # torch.matmul in the same round-robin: a number for scale, not a candidate
    log(f"{len(todo)} candidates to time, {len(done)} already in {out}")
    # Operands that fit the L2 are rotated over R copies so every launch streams from HBM, and each
    # candidate's launches are replayed as one CUDA graph: a call from Python costs more host time than
    # a small GEMM takes on the device.
    op_bytes = 2 * (M + N) * K
    rot = 1 if op_bytes > 252e6 else min(64, -(-512_000_000 // op_bytes))
    Bs = [Bt] + [Bt.clone() for _ in range(rot - 1)]
    reps = max(inner, 8, min(rot, 16))   # enough launches per replay for the first one's launch latency not to count
    side = torch.cuda.Stream()
    graphs = []
    for ov, p, ws, times in todo:
        with torch.cuda.stream(side):
            if p is None:
                torch.matmul(A, Bs[0].t())
            else:
                pkg.gemm(A, Bs[0], None, D, 1.0, 0.0, p, workspace=ws)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for i in range(reps):
                    if p is None:
                        torch.matmul(A, Bs[i % rot].t())
                    else:
                        pkg.gemm(A, Bs[i % rot], None, D, 1.0, 0.0, p, workspace=ws)
        graphs.append(g)
    for _ in range(rounds):
        for (ov, p, ws, times), g in zip(todo, graphs):
            with torch.cuda.stream(side):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                g.replay()
                e0.record(side)
                g.replay()
                e1.record(side)
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / reps)
    status, _ = pkg.device_status()
    with open(out, "a") as f:
        for ov, p, ws, times in todo:
            ms = sorted(times)[len(times) // 2]
            row = {"shape": [M, N, K], "dtype": dtype, "params": ov, "ms": ms, "tflops": 2.0 * M * N * K / (ms * 1e-3) / 1e12,
                   "gbs": (2.0 * (M * K + N * K) + 4.0 * M * N) / (ms * 1e-3) / 1e9, "status": status}
            f.write(json.dumps(row) + "\n")
    return best(out, M, N, K, dtype)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("M", type=int)
    ap.add_argument("N", type=int)
    ap.add_argument("K", type=int)
    ap.add_argument("--dtype", choices=["f16", "bf16"], default="f16")
    ap.add_argument("--out", default="tune.jsonl")
    ap.add_argument("--rounds", type=int, default=12)
    ap.add_argument("--with-library", action="store_true", help="time torch.matmul in the same round-robin, for scale")
    a = ap.parse_args()
    b = tune(a.M, a.N, a.K, a.dtype, a.out, a.rounds, with_library=a.with_library)
    print(json.dumps({"shape": [a.M, a.N, a.K], "dtype": a.dtype, "best": b}))
