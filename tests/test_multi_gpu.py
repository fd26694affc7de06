"""GPU, two or more devices: split-K over GPUs, with the exchange as an NCCL reduce-scatter and
fused into the GEMM epilogue (peer stores over NVLink), against the CPU oracle. One process per
GPU. Skipped on a single-GPU machine (tests/test_sharding.py covers the split logic on CPU)."""
import os
import sys

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
    from helpers import to_device, tolerance_ok
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
        out = torch.empty((m // world, n), dtype=torch.float32, device="cuda")
        for tile in (dict(tile_m=256, tile_n=256, cta_group=2), dict(tile_m=128, tile_n=128), dict(tile_m=256, tile_n=128, cta_group=2),
                     dict(tile_m=256, tile_n=256, cta_group=2, split_k=4), dict(tile_m=128, tile_n=256, split_k=3)):
            out.fill_(float("nan"))
            ex.gemm_reduce_scatter(dA, dB, out, pkg.default_params(m, n, ks.size, pkg.F16, **tile))
            torch.cuda.synchronize()
            results["fused " + str(tile)] = out.cpu().numpy().copy()
        st, info = pkg.device_status()
        ex.close()
        report = {name: tolerance_ok(got, want, k) for name, got in results.items()}
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
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, st, report in results:
        assert st == 0, (rank, st)
        for name, (ok, msg) in report.items():
            assert ok, (rank, name, msg)
