"""Launch timeline of the GEMM kernel: where the microseconds around the K loop go.

For steps of tens of microseconds (decode shapes) the time from kernel entry to the first load and
from the last MMA to exit is a visible share of the step. A diagnostic build of the library stamps
%globaltimer at set-up and role milestones of every CTA; this tool launches one GEMM, reads the
stamps back and prints, per milestone, mean / min / max over the working CTAs in nanoseconds from
the first CTA's entry.

    python cuda-kernel-opt_b200/build.py -DB200_TIMELINE --out cuda-kernel-opt_b200/libb200gemm_timeline.so
    B200_GEMM_LIB=cuda-kernel-opt_b200/libb200gemm_timeline.so python cuda-kernel-opt_b200/timeline.py 16 3584 8192

The reference times whole launches only (CUDA events, matmul_shmem_tc_async.cu:787-795). Needs a
B200; the operands of a small shape stay in L2 between launches, so the K-loop part of a timeline is
not an HBM measurement: use bench.py for that.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

MILESTONES = [
    (13, "kernel entry"),
    (16, "barriers initialised"),
    (17, "tensor memory allocated"),
    (14, "set-up barrier passed"),
    (27, "producer: preamble done"),
    (28, "producer: first unit decoded"),
    (19, "producer: first stage armed"),
    (20, "mma: first stage full"),
    (22, "epilogue: first accumulator ready"),
    (21, "mma: last tile committed"),
    (26, "epilogue: last accumulator ready"),
    (18, "epilogue: last tensor-memory load done"),
    (23, "epilogue: last stores issued"),
    (29, "epilogue: slice staged and announced (cluster reduce)"),
    (30, "epilogue: all slices ready (cluster reduce)"),
    (31, "epilogue: reduced columns stored (cluster reduce)"),
    (24, "epilogue: loop done"),
    (15, "exit"),
]


def summarise(stamps):
    """stamps: one row of %globaltimer values per CTA (nanoseconds, 0 = never stamped), at least 32 columns.
    Returns (CTAs entered, CTAs with work, rows) where rows = [(milestone, mean, min, max)] in nanoseconds
    from the first CTA's entry, over the CTAs that had work (an accumulator became ready); milestones no
    working CTA stamped are left out. Pure numpy: the part of the tool that needs no GPU."""
    import numpy as np
    r = np.asarray(stamps, dtype=np.int64)
    entered = r[:, 13] > 0
    if not entered.any():
        return 0, 0, []
    working = entered & (r[:, 22] > 0)
    t0 = int(r[entered, 13].min())
    rows = []
    for slot, name in MILESTONES:
        v = r[working, slot]
        v = v[v > 0] - t0
        if v.size == 0:
            continue
        rows.append((name, float(v.mean()), int(v.min()), int(v.max())))
    return int(entered.sum()), int(working.sum()), rows


def timeline(M: int, N: int, K: int, dtype: str = "bf16", overrides: dict | None = None, out=print):
    import torch
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    pkg = load_package()
    slots = pkg.profile_slots()
    if slots < 32:
        raise SystemExit("this library was built without -DB200_TIMELINE: see the commands at the top of this file")
    code = pkg.BF16 if dtype == "bf16" else pkg.F16
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float16
    A = torch.empty((M, K), dtype=tdt, device="cuda")
    Bt = torch.empty((N, K), dtype=tdt, device="cuda")
    pkg.fill_device(A, 2, 1)
    pkg.fill_device(Bt, 2, 2)
    D = torch.empty((M, N), dtype=torch.float32, device="cuda")
    p = pkg.default_params(M, N, K, code, **(overrides or {}))
    ctas = pkg.num_sms()
    prof = torch.zeros((ctas, slots), dtype=torch.int64, device="cuda")
    for _ in range(3):
        pkg.gemm(A, Bt, None, D, 1.0, 0.0, p)
    torch.cuda.synchronize()
    pkg.lib().b200_set_profile_buffer(prof.data_ptr(), ctas)
    pkg.gemm(A, Bt, None, D, 1.0, 0.0, p)
    torch.cuda.synchronize()
    pkg.lib().b200_set_profile_buffer(None, 0)
    st, info = pkg.device_status()
    entered, working, rows = summarise(prof.cpu().numpy())
    out(f"{M} x {N} x {K} {dtype}, params {p.as_dict()}")
    out(f"CTAs entered {entered}, with work {working}, device status {st}")
    for name, mean, lo, hi in rows:
        out(f"  {name:52s} mean {mean:9.0f} ns   min {lo:8d}   max {hi:8d}")
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("M", type=int)
    ap.add_argument("N", type=int)
    ap.add_argument("K", type=int)
    ap.add_argument("--dtype", choices=["f16", "bf16"], default="bf16")
    ap.add_argument("--params", default="", help="JSON overrides of the launch tunables")
    a = ap.parse_args()
    timeline(a.M, a.N, a.K, a.dtype, json.loads(a.params) if a.params else None)
