"""CPU: the multi-GPU split logic, including a world_size-2 gloo run of the split-K combine."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def shard_mod():
    import importlib
    from __graft_entry__ import load_package
    load_package()
    return importlib.import_module("cuda_kernel_opt_b200.shard")


def test_splits_cover_without_overlap():
    sh = shard_mod()
    for total, world, align in ((8192, 8, 128), (28672, 8, 224), (28672, 3, 256), (262144, 8, 64), (200, 4, 128), (64, 8, 64)):
        fn = {128: sh.m_shard, 224: sh.n_shard, 256: sh.n_shard, 64: sh.k_shard}[align]
        prev = 0
        for r in range(world):
            s = fn(total, world, r, align)
            assert s.begin == prev and s.begin <= s.end <= total
            assert s.begin % align == 0 and (s.end % align == 0 or s.end == total)
            prev = s.end
        assert prev == total
    with pytest.raises(ValueError):
        sh.m_shard(1024, 4, 4)


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        sh = shard_mod()
        m, n, k, seed = 64, 96, 512, 41
        A = oracle.fill_u16((m, k), seed, 1)
        Bt = oracle.fill_u16((n, k), seed, 2)
        # split-K: each rank multiplies its K slice (the CPU oracle stands in for the GPU kernel
        # here; the test is about the split and the combine), then reduce-scatter by rows
        ks = sh.k_shard(k, world, rank, 64)
        part = oracle.gemm(np.ascontiguousarray(A[:, ks.begin:ks.end]), np.ascontiguousarray(Bt[:, ks.begin:ks.end]))
        mine = sh.reduce_scatter_rows(torch.from_numpy(part)).numpy()
        full = oracle.gemm(A, Bt)
        rows = slice(rank * m // world, (rank + 1) * m // world)
        err_k = float(np.abs(mine - full[rows]).max())
        # M-shard and N-shard: no collective, the pieces tile the full product exactly
        ms = sh.m_shard(m, world, rank, 32)
        dm = oracle.gemm(np.ascontiguousarray(A[ms.begin:ms.end]), Bt)
        ns = sh.n_shard(n, world, rank, 16)
        dn = oracle.gemm(A, np.ascontiguousarray(Bt[ns.begin:ns.end]))
        exact = bool(np.array_equal(dm, full[ms.begin:ms.end]) and np.array_equal(dn, full[:, ns.begin:ns.end]))
        q.put((rank, err_k, exact, mine.shape))
    finally:
        dist.destroy_process_group()


def test_split_k_reduce_scatter_gloo_world2():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err_k, exact, shape in results:
        assert shape == (32, 96)
        assert err_k < 2.0 ** -10 * np.sqrt(512), (rank, err_k)   # split-K changes the summation order only
        assert exact, "M-/N-shards must reproduce the unsharded product bit for bit"


def _leaver(rank, world, port, q):
    """Rank 1 goes away between steps: once with a leave note, once silently. Rank 0 must learn of it on the
    host before its next launch (note), or have its next collective end with an error (short timeout)."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    sh = shard_mod()
    store = dist.distributed_c10d._get_default_store()
    out = {}
    try:
        mem = sh.Membership(store, rank, world, stale_after=1.0)
        x = torch.ones(4)
        dist.all_reduce(x)                                   # step 1: everybody is there
        out["step1"] = float(x[0])
        mem.beat(1)
        if rank == 1:
            mem.leave("planned exit after step 1")          # between steps, nothing in flight
            q.put((rank, out))
            return
        # rank 0: wait for the note (bounded), then check before "launching" step 2
        import time
        t0 = time.time()
        while time.time() - t0 < 20:
            try:
                mem.check()
            except sh.PeerLeft as e:
                out["left"] = (e.rank, e.reason)
                break
            time.sleep(0.05)
        # a heartbeat that stops: the same check with a clock that has moved on
        mem2 = sh.Membership(store, rank, world, prefix="b200/members2", stale_after=1.0)
        store.set("b200/members2/beat/1", f"1:{time.time() - 5.0:.3f}")
        try:
            mem2.check()
            out["stale"] = None
        except sh.PeerLeft as e:
            out["stale"] = (e.rank, "no heartbeat" in e.reason)
        # a peer gone without a note: the next collective ends with an error after the group's short timeout
        t0 = time.time()
        try:
            dist.all_reduce(x)
            out["collective"] = "returned"
        except Exception as e:       # gloo raises RuntimeError (timeout / connection closed by peer)
            out["collective"] = "error"
        out["collective_s"] = time.time() - t0
        q.put((rank, out))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_rank_leaving_between_steps_is_seen_on_the_host_gloo_world2():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_leaver, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert results[1]["step1"] == 2.0 and results[0]["step1"] == 2.0
    assert results[0]["left"] == (1, "planned exit after step 1")
    assert results[0]["stale"] == (1, True)
    assert results[0]["collective"] == "error" and results[0]["collective_s"] < 30
