"""GPU, two or more devices: split-K over GPUs, with the exchange as an NCCL reduce-scatter and
fused into the GEMM epilogue (peer stores over NVLink), against the CPU oracle. One process per
GPU. Skipped on a single-GPU machine (tests/test_sharding.py covers the split logic on CPU)."""
import os
import sys
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import importlib
    import torch
    import torch.distributed as dist
    import oracle
    from __graft_entry__ import load_package
    from helpers import Guarded, to_device, tolerance_ok
    pkg = load_package()
    shard = importlib.import_module("cuda_kernel_opt_b200.shard")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        m, n, k, seed = 256 * world, 512, 4096, 77
        A = pkg.fill_u16_host((m, k), seed, 1)
        Bt = pkg.fill_u16_host((n, k), seed, 2)
        ks = shard.k_shard(k, world, rank, 64)
        dA = to_device(torch, np.ascontiguousarray(A[:, ks.begin:ks.end]), pkg.F16)
        dB = to_device(torch, np.ascontiguousarray(Bt[:, ks.begin:ks.end]), pkg.F16)
        rows = slice(rank * m // world, (rank + 1) * m // world)
        want = oracle.gemm(A, Bt)[rows]
        results = {}
        # (1) GEMM, then NCCL reduce-scatter
        p = pkg.default_params(m, n, ks.size, pkg.F16, tile_m=256, tile_n=256, cta_group=2)
        part = pkg.gemm(dA, dB, params=p)
        results["nccl"] = shard.reduce_scatter_rows(part).cpu().numpy()
        # (2) exchange fused into the epilogue, three steps in a row (alternating slot areas)
        ex = shard.PushExchange(pkg, m, n)
        gout = Guarded(torch, (m // world, n), torch.float32)
        out = gout.t
        for tile in (dict(tile_m=256, tile_n=256, cta_group=2), dict(tile_m=128, tile_n=128), dict(tile_m=256, tile_n=128, cta_group=2),
                     dict(tile_m=256, tile_n=256, cta_group=2, split_k=4), dict(tile_m=128, tile_n=256, split_k=3)):
            out.fill_(float("nan"))
            ex.gemm_reduce_scatter(dA, dB, out, pkg.default_params(m, n, ks.size, pkg.F16, **tile))
            torch.cuda.synchronize()
            gout.check("rows of D, fused exchange " + str(tile))
            results["fused " + str(tile)] = out.cpu().numpy().copy()
        # (2b) one rank's host stalls between its push and its reduce while the others run on: they finish that
        # step and push the next one, so the late rank finds their flags one epoch ahead. Its reduce must take
        # that as "arrived" (the step's slots sit in the other area, untouched), not wait for an exact match.
        p_pair = pkg.default_params(m, n, ks.size, pkg.F16, tile_m=256, tile_n=256, cta_group=2)
        late = []
        for step in range(2):
            gout = Guarded(torch, (m // world, n), torch.float32)
            if rank == 0 and step == 0:
                ex.push(dA, dB, p_pair)
                torch.cuda.synchronize()
                time.sleep(0.6)
                ex.reduce(gout.t)
            else:
                ex.gemm_reduce_scatter(dA, dB, gout.t, p_pair)
            late.append(gout)
        torch.cuda.synchronize()
        for step, gout in enumerate(late):
            gout.check(f"rows of D, late-rank step {step}")
            results[f"fused, rank 0 late, step {step}"] = gout.t.cpu().numpy().copy()
        # (3) the shards that need no exchange, with default tunables: rows of B^T (columns of D) of a decode
        # shape per rank (swapped roles, K over a cluster), rows of A of a square per rank
        m2, n2, k2 = 16, 1024 * world, 4096
        A2, B2 = pkg.fill_u16_host((m2, k2), seed + 1, 1, dtype=pkg.BF16), pkg.fill_u16_host((n2, k2), seed + 1, 2, dtype=pkg.BF16)
        ns = shard.n_shard(n2, world, rank, 256)
        p2 = pkg.default_params(m2, ns.size, k2, pkg.BF16)
        assert p2.swap_ab == 1 and p2.cluster_reduce == 1
        got2 = pkg.gemm(to_device(torch, A2, pkg.BF16), to_device(torch, np.ascontiguousarray(B2[ns.begin:ns.end]), pkg.BF16), params=p2)
        want2 = oracle.gemm(A2, B2, dtype=oracle.BF16)[:, ns.begin:ns.end]
        m3, n3, k3 = 512 * world, 768, 1024
        A3, B3 = pkg.fill_u16_host((m3, k3), seed + 2, 1), pkg.fill_u16_host((n3, k3), seed + 2, 2)
        ms = shard.m_shard(m3, world, rank, 256)
        got3 = pkg.gemm(to_device(torch, np.ascontiguousarray(A3[ms.begin:ms.end]), pkg.F16), to_device(torch, B3, pkg.F16))
        want3 = oracle.gemm(A3, B3)[ms.begin:ms.end]
        # (4) the host-buffer call of an M-sharded square: B^T crosses PCIe once (every rank uploads its own rows and
        # copies them to the other GPUs over NVLink); two steps in a row with different operands
        m4, n4, k4 = 512, 512 * world, 1024
        hg = shard.HostGemmMShard(pkg, m4, n4, k4)
        host_reports = {}
        for step in range(2):
            A4 = pkg.fill_u16_host((m4 * world, k4), seed + 10 + step, 1)
            B4 = pkg.fill_u16_host((n4, k4), seed + 10 + step, 2)
            mine = np.ascontiguousarray(A4[rank * m4:(rank + 1) * m4])
            b_rows = np.ascontiguousarray(B4[rank * (n4 // world):(rank + 1) * (n4 // world)])
            out4 = np.full((m4, n4), np.nan, np.float32)
            hg.gemm(pkg.F16, mine, b_rows, None, out4, 1.0, 0.0)
            host_reports[f"host-buffer M-shard, step {step}"] = tolerance_ok(out4, oracle.gemm(mine, B4), k4)
        hg.close()
        torch.cuda.synchronize()
        st, info = pkg.device_status()
        ex.close()
        report = {name: tolerance_ok(got, want, k) for name, got in results.items()}
        report["N-shard, decode defaults"] = tolerance_ok(got2.cpu().numpy(), want2, k2)
        report["M-shard, defaults"] = tolerance_ok(got3.cpu().numpy(), want3, k3)
        report.update(host_reports)
        q.put((rank, st, report))
    finally:
        dist.destroy_process_group()


def test_split_k_over_gpus_nccl_and_fused():
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    import queue
    results, deadline = [], time.time() + 300
    while len(results) < world:
        try:
            results.append(q.get(timeout=2))
        except queue.Empty:
            dead = [p.exitcode for p in procs if p.exitcode not in (None, 0)]
            assert not dead, f"a rank exited with {dead} before reporting"       # fail at once, not after the time limit
            assert time.time() < deadline, "ranks did not report in time"
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, st, report in results:
        assert st == 0, (rank, st)
        for name, (ok, msg) in report.items():
            assert ok, (rank, name, msg)
