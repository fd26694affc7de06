"""Benchmark of the B200 asynchronous tensor-core GEMM (the hot path of this repository).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of synthetic input: one GEMM
D = A * B^T of the workload's shape. Default workload: the configuration the headline metric is
quoted on, M = N = K = 8192, fp16 inputs (uniform[-1,1), seed 2), fp32 accumulate and output.

N > 1 is launched by torch.distributed.run, one process per GPU. The default workload shards
along M with no collective, as the baseline states it: the 8192 rows of A and D are split into N
row blocks, one per GPU, B^T is replicated (strong scaling of one 8192^3 product; the line also
carries the per-GPU rate of a full 8192^3 on every GPU at once). `--scaling weak` gives every GPU
its own 8192-row block of a (8192*N)-row A instead. `--workload c5_splitk` is the one workload
with a real exchange step (fp32 reduce-scatter, fused into the GEMM epilogue over NVLink).

Rank 0 prints ONE JSON line. `value` is whole-job throughput with inputs resident in HBM;
`e2e` is the same metric through the host-buffer call of the C ABI (copies inside the timed
region); `roofline` is the kernel alone against the measured tensor peak; `cpu_baseline` is the
reference's own CPU matmul timed on this machine's host cores.

`--impl reference` times the reference's CPU implementation of the path (its host recompute
loop, compiled from its own header where available, else the CPU restatement) on a bounded sample
of the same workload, on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

# rank 0 prints exactly one line on stdout: keep NCCL's version banner off it
if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
    os.environ["NCCL_DEBUG"] = "WARN"

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fp16->fp32 GEMM TFLOPS at 8192^3 (whole job; per GPU = value / n_gpus)"
NOMINAL_TFLOPS = 2250.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM traffic of one launch of the dominant kernel from an ncu capture (dram__bytes_read.sum +
# dram__bytes_write.sum); see profiles/. None where no capture exists for the workload.
NCU_TRAFFIC_BYTES = {"c3_8192_f16": 939570688, "c2_4096_f16": 125323264, "c4_m16_bf16": 472698283, "c4_m128_bf16": 473866240}

WORKLOADS = {
    # name: (M, N, K, dtype, seed, dist_a, dist_b, bound)
    "c1_1024_f16": (1024, 1024, 1024, "f16", 0, (0, 1.0), (0, 1.0), "tensor"),
    "c2_4096_f16": (4096, 4096, 4096, "f16", 1, (0, 1.0), (0, 1.0), "tensor"),
    "c3_8192_f16": (8192, 8192, 8192, "f16", 2, (0, 1.0), (0, 1.0), "tensor"),
    "c3_8192_bf16": (8192, 8192, 8192, "bf16", 2, (0, 1.0), (0, 1.0), "tensor"),
    "c4_m16_bf16": (16, 28672, 8192, "bf16", 3, (1, 1.0), (1, 0.02), "hbm"),
    "c4_m128_bf16": (128, 28672, 8192, "bf16", 3, (1, 1.0), (1, 0.02), "hbm"),
    "c5_splitk_f16": (2048, 2048, 262144, "f16", 4, (0, 1.0), (0, 1.0), "tensor"),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons while the timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost"}

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.stop_flag, self.sm, self.bits, self.max_sm, self.power = index, False, [], 0, None, []
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def sample(self):
        if self.nv is None:
            return
        try:
            self.sm.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            if len(self.sm) % 8 == 1:
                self.power.append(self.nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            try:
                self.bits |= self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            except Exception:
                self.bits |= self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        except Exception:
            pass

    def run(self):
        while not self.stop_flag:
            self.sample()
            time.sleep(0.0005)

    def energy_mj(self):
        """Total energy the GPU has drawn since the driver loaded, in millijoules (read-only NVML counter), or None."""
        if self.nv is None:
            return None
        try:
            return int(self.nv.nvmlDeviceGetTotalEnergyConsumption(self.h))
        except Exception:
            return None

    def summary(self):
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None,
                "sm_max_mhz": self.max_sm, "power_w_max": max(self.power) if self.power else None, "samples": len(sm),
                "reasons": [name for bit, name in self.REASONS.items() if self.bits & bit]}


def bind_to_gpu_numa_node(index: int):
    """Runs this process on the CPUs next to its GPU (NVML's affinity mask), so that the pinned host buffers it
    allocates afterwards are placed in that socket's memory and host <-> device copies do not cross sockets.
    Read-only with respect to the GPU; a no-op where NVML or the affinity call is unavailable."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
        return sorted(cpus)
    except Exception:
        return None


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def flops_of(m, n, k):
    return 2.0 * m * n * k


def bytes_of(m, n, k):
    return 2.0 * (m * k + n * k) + 4.0 * m * n


# ---------------------------------------------------------------------------------------------
# reference arm: the reference's CPU matmul on the host cores
# ---------------------------------------------------------------------------------------------

def cpu_reference_rate(workload: str, seconds_budget: float, steps: int = 1, warmup: int = 0, all_threads: bool = False):
    """Times the reference's host recompute (GetNumIncorrect, matmul_test.h:307-326, through
    oracle/_ref) or, where that library is absent, the CPU restatement, on a slab of rows of the
    workload. Returns (tflops, info dict, ms_per_step)."""
    import numpy as np
    import oracle
    M, N, K, dts, seed, da, db, _ = WORKLOADS[workload]
    dtype = oracle.BF16 if dts == "bf16" else oracle.FP16
    use_ref = oracle.have_ref() and N == K          # the reference reads B^T with pitch n: square only
    threads = 1
    if all_threads:
        threads = max(1, os.cpu_count() or 1)
        if use_ref:
            # one instance of the reference's fixture class per thread, each holding A, B, C and the result at
            # N x N (4 + 12 bytes per element): use every core that memory allows
            per_instance = 12.5 * N * N
            try:
                import psutil
                threads = max(1, min(threads, int(0.5 * psutil.virtual_memory().available / per_instance)))
            except Exception:
                threads = min(threads, 8)
    Bt = oracle.fill_u16((N, K), seed, oracle.TENSOR_B, int(db[0]), float(db[1]), dtype)
    if use_ref:
        rate_guess = 0.6e9                           # flop/s of the scalar loop on one core
        rows = int(max(1, min(M, seconds_budget * rate_guess / (2.0 * N * K) / max(1, steps + warmup))))
        A = oracle.fill_u16((rows * threads, K), seed, oracle.TENSOR_A, int(da[0]), float(da[1]), dtype)
        res = np.zeros((rows, N), np.float32)
        sessions = [None] * threads

        def make(t):                                 # the fixture's constructor fills four N x N arrays: in parallel
            s = oracle.RefSession(N, dtype)
            s.load(np.ascontiguousarray(A[t * rows:(t + 1) * rows]), Bt, None)
            sessions[t] = s
        makers = [threading.Thread(target=make, args=(t,)) for t in range(threads)]
        for t in makers:
            t.start()
        for t in makers:
            t.join()

        def step():
            if threads == 1:
                sessions[0].count_incorrect(res, 1.0, 0.0, 0.1)
            else:
                ts = [threading.Thread(target=s.count_incorrect, args=(res, 1.0, 0.0, 0.1)) for s in sessions]
                for t in ts:
                    t.start()
                for t in ts:
                    t.join()
        kind = "reference"
    else:
        rate_guess = 2.5e9 * threads
        rows = int(max(1, min(M, seconds_budget * rate_guess / (2.0 * N * K) / max(1, steps + warmup))))
        A = oracle.fill_u16((rows, K), seed, oracle.TENSOR_A, int(da[0]), float(da[1]), dtype)

        def step():
            oracle.gemm(A, Bt, None, 1.0, 0.0, dtype, threads=threads)
        kind = "port"
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(max(1, steps)):
        step()
    dt = (time.perf_counter() - t0) / max(1, steps)
    total_rows = rows * (threads if use_ref else 1)
    tflops = flops_of(total_rows, N, K) / dt / 1e12
    for s in (sessions if use_ref else []):
        s.close()
    info = {"value": tflops, "unit": "TFLOPS", "cores": threads, "host_cores": os.cpu_count(), "kind": kind,
            "sample": f"{total_rows} of {M} rows of D (all {N} columns, K = {K}) per step, "
                      f"{'the reference GetNumIncorrect loop (matmul_test.h:307-326)' if use_ref else 'CPU restatement of that loop'}"}
    return tflops, info, dt * 1e3


def run_reference_arm(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return 0
    M, N, K, dts, *_ = WORKLOADS[args.workload]
    tflops, info, ms = cpu_reference_rate(args.workload, seconds_budget=40.0, steps=args.steps, warmup=args.warmup, all_threads=True)
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOPS", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16" if dts == "f16" else "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "M": M, "N": N, "K": K, "device": "host CPU", "sample": info["sample"]},
        "cpu_baseline": info,
        "e2e": {"value": tflops, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------

def run_ours(args):
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    import importlib
    shard = importlib.import_module("cuda_kernel_opt_b200.shard")

    rank, world, local = dist_env()
    if world != args.gpus and world > 1:
        args.gpus = world
    assert torch.cuda.is_available(), "bench.py --impl ours needs a GPU: the library has no CPU path"
    torch.cuda.set_device(local)
    bind_to_gpu_numa_node(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    M, N, K, dts, seed, da, db, bound = WORKLOADS[args.workload]
    dtype = pkg.BF16 if dts == "bf16" else pkg.F16
    tdt = torch.bfloat16 if dts == "bf16" else torch.float16
    splitk_ranks = args.workload.startswith("c5") and world > 1
    nshard = args.workload.startswith("c4")

    # --shard-of G on one GPU: time rank 0's shard of a G-GPU run of an N-sharded workload alone
    mshard_alone = args.shard_of > 1 and world == 1 and not nshard and not args.workload.startswith("c5")
    shard_world = args.shard_of if (args.shard_of > 1 and world == 1 and (nshard or mshard_alone)) else world
    library = args.impl == "library"       # torch.matmul (cuBLAS) in the same harness, for scale only
    # the library's product: fp16/bf16 out by default (torch.matmul); --library-out f32 asks it for this path's fp32 D
    if args.library_out == "f32":
        lib_mm = lambda a_, bt_: torch.mm(a_, bt_.t(), out_dtype=torch.float32)
    else:
        lib_mm = lambda a_, bt_: torch.matmul(a_, bt_.t())

    # ---- placement (see cuda-kernel-opt_b200/shard.py)
    if splitk_ranks:                         # K split over ranks, fp32 partials reduce-scattered by rows
        ks = shard.k_shard(K, world, rank, 64)
        m_loc, n_loc, k_loc = M, N, ks.size
        a_begin, b_begin, a_pitch = ks.begin, ks.begin, K
        scaling, parallelism = "strong", f"split-K x{world} + NCCL reduce-scatter"
    elif nshard:                             # rows of B^T (weights) split over ranks, activations replicated
        ns = shard.n_shard(N, shard_world, rank, 256)
        m_loc, n_loc, k_loc = M, ns.size, K
        scaling, parallelism = "strong", f"N-shard x{shard_world}, no collective" + (" (rank 0's shard alone on one GPU)" if shard_world != world else "")
    elif args.scaling == "strong":           # rows of A split over ranks, B^T replicated
        ms = shard.m_shard(M, shard_world, rank, 256)
        m_loc, n_loc, k_loc = ms.size, N, K
        scaling, parallelism = "strong", f"M-shard x{shard_world}, no collective" + (" (rank 0's shard alone on one GPU)" if shard_world != world else "")
    else:                                    # every rank owns a full M-row block of a (M*world)-row A
        m_loc, n_loc, k_loc = M, N, K
        scaling, parallelism = "weak", f"M-shard x{world} ({M} rows per GPU), no collective"

    # ---- synthetic operands, generated on the device by the seeded generator
    A = torch.empty((m_loc, k_loc), dtype=tdt, device=dev)
    Bt = torch.empty((n_loc, k_loc), dtype=tdt, device=dev)
    if splitk_ranks:
        # a K slice is strided in the full operand: generate row by row ranges
        for r0 in range(0, M, 256):
            rows = min(256, M - r0)
            tmp = torch.empty((rows, K), dtype=tdt, device=dev)
            pkg.fill_device(tmp, seed, 1, int(da[0]), float(da[1]), begin=r0 * K)
            A[r0:r0 + rows].copy_(tmp[:, ks.begin:ks.end])
            pkg.fill_device(tmp, seed, 2, int(db[0]), float(db[1]), begin=r0 * K)
            Bt[r0:r0 + rows].copy_(tmp[:, ks.begin:ks.end])
        del tmp
    else:
        a_row0 = (rank * M if (scaling == "weak") else (shard.m_shard(M, shard_world, rank, 256).begin if not nshard else 0))
        b_row0 = shard.n_shard(N, shard_world, rank, 256).begin if nshard else 0
        pkg.fill_device(A, seed, 1, int(da[0]), float(da[1]), begin=a_row0 * K)
        pkg.fill_device(Bt, seed, 2, int(db[0]), float(db[1]), begin=b_row0 * K)
    D = torch.empty((m_loc, n_loc), dtype=torch.float32, device=dev)
    # Operands that would stay in the 126 MB L2 between steps are rotated: R identical copies, step i
    # reads copy i mod R, so every step streams its operands from HBM.
    op_bytes = 2 * (m_loc * k_loc + n_loc * k_loc)
    rot = 1 if op_bytes > 252e6 else min(64, -(-512_000_000 // op_bytes))
    As = [A] + [A.clone() for _ in range(rot - 1)]
    Bts = [Bt] + [Bt.clone() for _ in range(rot - 1)]

    overrides = json.loads(args.params) if args.params else {}
    fused = splitk_ranks and args.exchange == "fused"
    if args.workload.startswith("c5") and not overrides:
        # 64 tiles of 256 x 256 on 74 CTA pairs: split K inside the GPU so every pair has equal work
        overrides = {"cta_group": 2, "split_k": 8}
    p = pkg.default_params(m_loc, n_loc, k_loc, dtype, **overrides)
    st = pkg.validate(m_loc, n_loc, k_loc, dtype, p)
    assert st == pkg.OK, f"invalid configuration {p.as_dict()}: {pkg.status_string(st)}"
    ws_bytes = pkg.workspace_bytes(m_loc, n_loc, k_loc, p)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    # the split-K reduce is a second kernel (not with the cluster reduce; the tail split finishes inside the GEMM)
    launches_per_step = 1 + (1 if (p.split_k > 1 and not p.cluster_reduce) else 0) + (1 if fused else 0)
    push = shard.PushExchange(pkg, M, N) if fused else None
    D_rows = torch.empty((M // world, N), dtype=torch.float32, device=dev) if fused else None
    if fused:
        parallelism = f"split-K x{world}, reduce-scatter fused into the epilogue (NVLink peer stores)"

    def step(i=0):
        a_i, b_i = As[i % rot], Bts[i % rot]
        if fused:
            return push.gemm_reduce_scatter(a_i, b_i, D_rows, p, workspace=ws if ws_bytes else None)
        if library:
            return lib_mm(a_i, b_i)
        pkg.gemm(a_i, b_i, None, D, 1.0, 0.0, p, workspace=ws if ws_bytes else None)
        if splitk_ranks:
            return shard.reduce_scatter_rows(D)
        return None

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: W warm-up steps, then exactly K timed steps
    for i in range(max(args.warmup, 3)):
        step(i)
    st, info = pkg.device_status()
    assert st == pkg.OK, f"device status {st} {info}"
    sampler = ClockSampler(local)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(args.steps)]
    # Steps of the order of a host launch (expected device time under 0.3 ms: the decode shapes and the
    # small squares, not 8192^3) are issued as one CUDA graph of the K steps, the way a serving loop
    # issues them, so the device is timed and not the Python interpreter; --graph 0/1 overrides.
    short_step = max(flops_of(m_loc, n_loc, k_loc) / 1.4e15, bytes_of(m_loc, n_loc, k_loc) / 6.0e12) < 0.3e-3
    use_graph = (short_step and not splitk_ranks) if args.graph < 0 else bool(args.graph)
    graph = None
    if use_graph:
        cap = torch.cuda.Stream(dev)
        cap.wait_stream(torch.cuda.current_stream(dev))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(cap):
            with torch.cuda.graph(graph, stream=cap):
                for i in range(args.steps):
                    step(i)
            graph.replay()                             # one untimed replay: graph upload
        torch.cuda.synchronize()
    barrier()
    sampler.start()
    if graph is not None:
        with torch.cuda.stream(cap):
            ev[0][0].record()
            graph.replay()
            ev[-1][2].record()
    else:
        for i, (e0, e1, e2) in enumerate(ev):
            a_i, b_i = As[i % rot], Bts[i % rot]
            e0.record()
            if fused:
                push.gemm_reduce_scatter(a_i, b_i, D_rows, p, workspace=ws if ws_bytes else None)
                e1.record()
            else:
                if library:
                    lib_mm(a_i, b_i)
                else:
                    pkg.gemm(a_i, b_i, None, D, 1.0, 0.0, p, workspace=ws if ws_bytes else None)
                e1.record()                                # end of the GEMM kernel(s) of this step
                if splitk_ranks:
                    shard.reduce_scatter_rows(D)
            e2.record()
    barrier()
    sampler.stop_flag = True
    sampler.join()
    total_ms = ev[0][0].elapsed_time(ev[-1][2])
    if graph is not None:
        kernel_ms, exposed_ms = total_ms / args.steps, 0.0
    else:
        kernel_ms = sum(e0.elapsed_time(e1) for e0, e1, _ in ev) / args.steps
        exposed_ms = sum(e1.elapsed_time(e2) for _, e1, e2 in ev) / args.steps
    st, info = pkg.device_status()
    assert st == pkg.OK, f"device status {st} {info}"
    step_ms = None if graph is not None else [round(e0.elapsed_time(e1), 5) for e0, e1, _ in ev]
    t = torch.tensor([total_ms, kernel_ms, exposed_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, kernel_ms, exposed_ms = (float(x) for x in t.tolist())
    ms_per_step = total_ms / args.steps

    # ---- N > 1, strong scaling of a square workload: the per-GPU rate when every GPU multiplies a full
    # M x N x K at the same time (what `--scaling weak` times), as an extra key beside the sharded number
    weak_extra = None
    if world > 1 and scaling == "strong" and not nshard and not splitk_ranks and not library:
        A_full = torch.empty((M, K), dtype=tdt, device=dev)
        pkg.fill_device(A_full, seed, 1, int(da[0]), float(da[1]), begin=0)
        D_full = torch.empty((M, N), dtype=torch.float32, device=dev)
        p_full = pkg.default_params(M, N, K, dtype)
        ws_full = torch.empty(max(pkg.workspace_bytes(M, N, K, p_full), 16), dtype=torch.uint8, device=dev)
        for _ in range(3):
            pkg.gemm(A_full, Bt, None, D_full, 1.0, 0.0, p_full, workspace=ws_full)
        barrier()
        w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0.record()
        for _ in range(args.steps):
            pkg.gemm(A_full, Bt, None, D_full, 1.0, 0.0, p_full, workspace=ws_full)
        w1.record()
        barrier()
        tw = torch.tensor([w0.elapsed_time(w1) / args.steps], dtype=torch.float64, device=dev)
        dist.all_reduce(tw, op=dist.ReduceOp.MAX)
        per_gpu = flops_of(M, N, K) / (float(tw.item()) * 1e-3) / 1e12
        weak_extra = {"what": f"every GPU multiplies its own {M} x {N} x {K} at the same time (--scaling weak)",
                      "ms_per_step": float(tw.item()), "per_gpu_tflops": per_gpu, "box_tflops": per_gpu * world}
        del A_full, D_full, ws_full

    # ---- the loaded state: seconds of back-to-back launches with clock, power and energy readings
    # (the timed region above is over before the power limit settles or NVML takes a sample under load)
    sustained = None
    if args.sustained_seconds > 0 and not short_step and not splitk_ranks and bound == "tensor":
        def sustained_leg(fn, leg_flops):
            smp = ClockSampler(local)
            chunk = max(1, int(0.02 / max(kernel_ms * 1e-3, 1e-5)))
            marks = []
            torch.cuda.synchronize()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            en0 = smp.energy_mj()
            smp.start()
            t_host = time.perf_counter()
            s0.record()
            n = 0
            while time.perf_counter() - t_host < args.sustained_seconds:
                for _ in range(chunk):
                    fn(n)
                    n += 1
                mk = torch.cuda.Event()
                mk.record()
                marks.append(mk)
                if len(marks) > 2:                      # at most two chunks queued ahead of the device
                    marks.pop(0).synchronize()
            s1.record()
            torch.cuda.synchronize()
            en1 = smp.energy_mj()
            smp.stop_flag = True
            smp.join()
            ms = s0.elapsed_time(s1)
            c = smp.summary()
            joules = (en1 - en0) / 1e3 if (en0 is not None and en1 is not None) else None
            tf = leg_flops * n / (ms * 1e-3) / 1e12
            return {"seconds": ms / 1e3, "launches": n, "tflops": tf, "ms_per_launch": ms / n,
                    "sm_mhz_median": c["sm_mhz"], "sm_mhz_min": c["sm_min_mhz"], "reasons": c["reasons"],
                    "ms_x_mhz": (ms / n) * c["sm_mhz"] if c["sm_mhz"] else None,
                    "power_w_mean": (joules / (ms / 1e3)) if joules is not None else None,
                    "joules_per_tflop": (joules / (leg_flops * n / 1e12)) if joules is not None else None}

        if library:
            sustained = sustained_leg(lambda i: lib_mm(As[i % rot], Bts[i % rot]), flops_of(m_loc, n_loc, k_loc))
        else:
            # the vendor library in the same harness, same duration, directly after (or, --sustained-library-first,
            # directly before: the second leg starts on a warmer GPU): a number for scale (joules per TFLOP side by
            # side); it is not on this repository's path
            lib_leg = None
            with_lib = world == 1 and rank == 0
            if with_lib and args.sustained_library_first:
                lib_leg = sustained_leg(lambda i: lib_mm(As[i % rot], Bts[i % rot]), flops_of(m_loc, n_loc, k_loc))
            sustained = sustained_leg(lambda i: pkg.gemm(As[i % rot], Bts[i % rot], None, D, 1.0, 0.0, p, workspace=ws if ws_bytes else None),
                                      flops_of(m_loc, n_loc, k_loc))
            st, info = pkg.device_status()
            assert st == pkg.OK, f"device status {st} {info}"
            if with_lib and lib_leg is None:
                lib_leg = sustained_leg(lambda i: lib_mm(As[i % rot], Bts[i % rot]), flops_of(m_loc, n_loc, k_loc))
            if lib_leg is not None:
                lib_leg["order"] = "before this kernel's leg" if args.sustained_library_first else "after this kernel's leg"
                sustained["library_for_scale"] = lib_leg
        sustained["frac_of_sustained_peak"] = sustained["tflops"] / peaks()["bf16_tflops_sustained"]
        sustained["peak_source"] = f"{peaks()['_source']} cuBLAS bf16 8192^3 sustained"

    job_flops = flops_of(M, N, K) * (world if scaling == "weak" else 1)
    job_bytes = bytes_of(M, N, K) * (world if scaling == "weak" else 1)
    if shard_world != world:                 # one shard alone: report the shard's own rate
        job_flops, job_bytes = flops_of(m_loc, n_loc, k_loc), bytes_of(m_loc, n_loc, k_loc)
    if bound == "tensor":
        value, unit = job_flops / (ms_per_step * 1e-3) / 1e12, "TFLOPS"
    else:
        value, unit = job_bytes / (ms_per_step * 1e-3) / 1e9, "GB/s"

    # ---- roofline of the dominant kernel (per GPU): algorithmic work of one launch / its duration
    pk = peaks()
    launch_flops, launch_bytes = flops_of(m_loc, n_loc, k_loc), bytes_of(m_loc, n_loc, k_loc)
    ncu_traffic = NCU_TRAFFIC_BYTES.get(args.workload) if (m_loc, n_loc, k_loc) == (M, N, K) else None   # captured on the whole shape only
    long_run = total_ms > 1000.0
    if bound == "tensor":
        achieved = launch_flops / (kernel_ms * 1e-3) / 1e12
        peak = pk["bf16_tflops_sustained"] if long_run else pk["bf16_tflops"]
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": ncu_traffic, "traffic_source": "ncu capture of one launch of this workload, profiles/ (not a value of this run)",
                "kernel": "gemm_sm100_kernel", "kernel_ms": kernel_ms,
                "peak_source": f"{pk['_source']} cuBLAS bf16 8192^3, {'sustained' if long_run else 'burst'}",
                "frac_of_nominal_2250": achieved / NOMINAL_TFLOPS, "algorithmic_flops_per_launch": launch_flops}
    else:
        achieved = launch_bytes / (kernel_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                "traffic": ncu_traffic, "kernel": "gemm_sm100_kernel", "kernel_ms": kernel_ms,
                "peak_source": f"{pk['_source']} copy bandwidth", "algorithmic_bytes_per_launch": launch_bytes}

    # ---- end to end: the host-buffer call of the C ABI (H2D of A, B^T, launch, D2H of D, sync)
    e2e = None
    if not splitk_ranks and not args.no_e2e and not library:
        sharded_host = world > 1 and scaling == "strong" and not nshard and N % world == 0 and (N // world) % 256 == 0
        hA = torch.empty((m_loc, k_loc), dtype=tdt).pin_memory()
        hD = torch.empty((m_loc, n_loc), dtype=torch.float32).pin_memory()
        hA.copy_(A)
        e_steps = max(1, min(args.steps, 10))
        if sharded_host:
            # M-shard on several GPUs: B^T crosses PCIe once. Every rank uploads its rows of A and only its N / world
            # rows of B^T, the GPUs exchange the B^T rows over NVLink (peer copies), every rank downloads its rows of D.
            rows_b = N // world
            hB = torch.empty((rows_b, k_loc), dtype=tdt).pin_memory()
            hB.copy_(Bt[rank * rows_b:(rank + 1) * rows_b])
            hg = shard.HostGemmMShard(pkg, m_loc, N, K)
            run_e2e = lambda: hg.gemm(dtype, hA, hB, None, hD, 1.0, 0.0)
            h2d = int(2 * (m_loc * k_loc + rows_b * k_loc))
            call = ("b200_session_gemm_host_sharded (pinned host rows of A and N / world rows of B^T -> device, B^T rows exchanged "
                    "between the GPUs over NVLink, one product per column block, rows of D -> pinned host, synchronised)")
        else:
            hB = torch.empty((n_loc, k_loc), dtype=tdt).pin_memory()
            hB.copy_(Bt)
            sess = pkg.Session(m_loc, n_loc, k_loc)
            p_host = p if p.split_k == 1 else None
            run_e2e = lambda: sess.gemm_host(dtype, hA, hB, None, hD, 1.0, 0.0, m_loc, n_loc, k_loc, p_host)
            h2d = int(2 * (m_loc * k_loc + n_loc * k_loc))
            call = ("b200_session_gemm_host (pinned host A, B^T -> device, GEMM, D -> pinned host, synchronised; A and B^T uploaded in "
                    "eight row blocks each, the band of D every block completes multiplied and downloaded at once: upload / compute / "
                    "download streams)")
        run_e2e()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e_steps):
            run_e2e()
        dt = (time.perf_counter() - t0) / e_steps
        tt = torch.tensor([dt], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
        ev_ = (job_flops / dt / 1e12) if bound == "tensor" else (job_bytes / dt / 1e9)
        pkg.gemm(A, Bt, None, D, 1.0, 0.0, p, workspace=ws if ws_bytes else None)     # the device-resident result of the same operands
        torch.cuda.synchronize()
        diff = float((hD.to(dev) - D).abs().max())
        st, info = pkg.device_status()
        assert st == pkg.OK, f"device status {st} {info}"
        bound_abs = 2.0 ** -10 * (k_loc ** 0.5) * (1.0 if int(da[0]) == 0 else 16.0)
        e2e = {"value": ev_, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(4 * m_loc * n_loc), "steps": e_steps,
               "ms_per_step": dt * 1e3, "call": call, "result_equals_device_run": diff == 0.0,
               "result_max_abs_diff_vs_device_run": diff, "result_within_tolerance_of_device_run": diff <= bound_abs,
               "note": "the host-buffer call multiplies block by block; a block product and the whole product visit their tiles in "
                       "another order, and the K order of a tile (k_order) and the tiles the tail split cuts follow that order: "
                       "differences are fp32 summation order, bounded by the stated per-element tolerance 2^-10 * sqrt(K)"}
        if sharded_host:
            hg.close()
        else:
            sess.close()
        del hA, hB, hD

    # ---- optional: per-role cycle counters of CTA 0 from one extra launch (tracing hook of the library)
    roles = None
    if args.role_counters and rank == 0:
        nblk = args.role_block + 1
        prof = torch.zeros((nblk, pkg.profile_slots()), dtype=torch.int64, device=dev)
        pkg.lib().b200_set_profile_buffer(prof.data_ptr(), nblk)
        pkg.gemm(A, Bt, None, D, 1.0, 0.0, p, workspace=ws if ws_bytes else None)
        torch.cuda.synchronize()
        pkg.lib().b200_set_profile_buffer(None, 0)
        r = prof.cpu().tolist()[args.role_block]
        it, tiles = max(r[9], 1), max(r[12], 1)
        roles = {"block": args.role_block, "stages": r[9], "units": r[12], "producer_cycles_per_stage": r[1] / max(r[2], 1),
                 "producer_wait_per_stage": r[0] / max(r[2], 1), "mma_cycles_per_stage": r[8] / it,
                 "mma_wait_data_per_stage": r[6] / it, "mma_wait_accumulator_per_unit": r[7] / tiles,
                 "mma_wait_accumulator_total": r[7], "mma_cycles_total": r[8],
                 "epilogue_cycles_per_unit": r[11] / tiles, "epilogue_wait_per_unit": r[10] / tiles,
                 "epilogue_cycles_total": r[11], "epilogue_wait_total": r[10], "kernel_ns": r[15] - r[13],
                 "stages_started_before_last_rows_of_a": r[-2]}

    # ---- CPU baseline beside it (rank 0, N = 1 only, bounded sample)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        _, cpu, _ = cpu_reference_rate(args.workload, seconds_budget=args.cpu_seconds)

    # ---- optional reported baseline: the reference's own WMMA kernel recompiled for sm_100a
    wmma = None
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_wmma_async")
    want_wmma = args.wmma_baseline == 1 or (args.wmma_baseline < 0 and os.path.exists(exe) and not library)
    if want_wmma and rank == 0 and world == 1 and M == N == K:
        if os.path.exists(exe):
            import subprocess
            r = subprocess.run([exe, str(M), "128", "64", "1", "3", "4", "8", "2"], capture_output=True, text=True, timeout=600)
            try:
                wmma = json.loads(r.stdout.strip().splitlines()[-1])
                wmma["what"] = "gemm_shmem_tc_async<half,float> of the reference (matmul_shmem_tc_async.cu), nvcc -arch=sm_100a, tile 128, seg_k 64, 3 stages, 4+8 warps"
            except Exception:
                wmma = {"error": (r.stdout + r.stderr)[-300:]}
        else:
            wmma = {"unavailable": "oracle/_ref/ref_wmma_async not built (make -C oracle wmma, needs the reference tree)"}

    if library:
        e2e = None
    if rank == 0:
        line = {
            "metric": METRIC if args.workload == "c3_8192_f16" else f"{unit} on {args.workload}",
            "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": dts, "data": "synthetic",
            "config": {"workload": args.workload, "M": M, "N": N, "K": K, "per_gpu": [m_loc, n_loc, k_loc],
                       "parallelism": parallelism, "alpha": 1.0, "beta": 0.0,
                       "l2": "inputs exceed twice the L2 (no flush needed)" if rot == 1 else
                             f"{rot} operand copies used in rotation ({rot * op_bytes / 1e6:.0f} MB): every step streams from HBM",
                       "issue": "one CUDA graph of the timed steps" if graph is not None else "one library call per step",
                       "params": p.as_dict(), "seed": seed},
            "roofline": roof, "cpu_baseline": cpu, "clocks": sampler.summary(), "e2e": e2e,
            "gpu_launches": args.steps * launches_per_step,
            "per_gpu_tflops": (value / world) if unit == "TFLOPS" else None,
        }
        if library:
            line["impl"] = "library (torch.matmul, for scale: not this repository's kernel)"
            line["library_out"] = args.library_out
            line["gpu_launches"] = 0
            line["config"].pop("params", None)
        if step_ms is not None:
            line["step_ms"] = step_ms
        if sustained:
            line["sustained"] = sustained
        if weak_extra:
            line["weak_scaling"] = weak_extra
        line["host_cores"] = os.cpu_count()
        if roles:
            line["role_counters"] = roles
        if wmma:
            line["reference_wmma_kernel"] = wmma
        if splitk_ranks:
            line["exposed_reduce_ms"] = exposed_ms
        print(json.dumps(line), flush=True)
    if fused and args.check:
        pkg.gemm(A, Bt, None, D, 1.0, 0.0, p)
        want = shard.reduce_scatter_rows(D)
        got = push.gemm_reduce_scatter(A, Bt, D_rows, p)
        torch.cuda.synchronize()
        rel = float((got - want).norm() / want.norm())
        st, info = pkg.device_status()
        print(f"[rank {rank}] fused vs NCCL reduce-scatter: rel diff {rel:.3e}, device status {st}", file=sys.stderr, flush=True)
    if push is not None:
        push.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference", "library"], default="ours",
                    help="library: torch.matmul in this harness, a number for scale (single-process workloads only)")
    ap.add_argument("--shard-of", type=int, default=0, help="one GPU: time rank 0's shard of a G-GPU run (N-shard of the decode workloads, M-shard of the squares)")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="c3_8192_f16")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="strong",
                    help="N > 1, square workloads: strong = the workload's M rows split over the GPUs (the baseline's "
                         "configuration), weak = every GPU gets M rows of its own")
    ap.add_argument("--library-out", choices=["half", "f32"], default="half",
                    help="what the vendor library writes where it is timed for scale: its default 16-bit D, or fp32 like this path (torch.mm out_dtype)")
    ap.add_argument("--sustained-library-first", action="store_true", help="run the vendor library's sustained leg before this kernel's instead of after")
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="after the timed steps, this many seconds of back-to-back launches with clock, power and energy "
                         "readings (0 = skip)")
    ap.add_argument("--exchange", choices=["nccl", "fused"], default="fused",
                    help="split-K workloads on N > 1: NCCL reduce-scatter after the GEMM, or fused into its epilogue")
    ap.add_argument("--check", action="store_true", help="split-K workloads: compare fused and NCCL results")
    ap.add_argument("--params", default="", help="JSON overrides of the launch tunables")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--graph", type=int, default=-1, help="1: issue the timed steps as one CUDA graph, 0: one call per step; default: graph when a step is expected to take under 0.3 ms")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--wmma-baseline", type=int, default=-1,
                    help="time the reference's own WMMA kernel recompiled for sm_100a (oracle/_ref/ref_wmma_async) beside "
                         "the number: 1 = yes, 0 = no, default = yes on one GPU when the binary is there")
    ap.add_argument("--role-counters", action="store_true", help="add in-kernel per-role cycle counters of one CTA")
    ap.add_argument("--role-block", type=int, default=0, help="which CTA the role counters come from")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
