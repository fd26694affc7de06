"""CPU: the sweep harness's candidate generation, JSONL record and resume logic (no timing here), and the
stamp arithmetic of the launch-timeline tool."""
import importlib
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def tune_mod():
    from __graft_entry__ import load_package
    load_package()
    return importlib.import_module("cuda_kernel_opt_b200.tune")


def test_candidates_are_valid_or_filtered(pkg):
    t = tune_mod()
    for shape in ((8192, 8192, 8192), (16, 28672, 8192), (128, 3584, 8192), (2048, 2048, 262144), (1024, 1024, 1024)):
        cands = t.candidates(*shape)
        assert len(cands) >= 8 and len({t.key_of(c) for c in cands}) == len(cands)
        valid = [c for c in cands if pkg.validate(*shape, pkg.F16, pkg.default_params(*shape, pkg.F16, **c)) == pkg.OK]
        assert len(valid) >= len(cands) // 2, shape
    assert any(c.get("split_k", 1) > 1 for c in t.candidates(2048, 2048, 262144))      # too few tiles: split-K offered
    skinny = t.candidates(16, 3584, 8192)
    assert any(c.get("swap_ab") and c.get("cluster_reduce") for c in skinny)            # decode shard: cluster over K offered
    assert all(pkg.validate(16, 3584, 8192, pkg.BF16, pkg.default_params(16, 3584, 8192, pkg.BF16, **c)) == pkg.OK
               for c in skinny if c.get("swap_ab"))
    assert not any(c.get("split_k", 1) > 1 for c in t.candidates(8192, 8192, 8192))


def test_record_resume_and_best(tmp_path):
    t = tune_mod()
    path = str(tmp_path / "tune.jsonl")
    rows = [{"shape": [64, 64, 64], "dtype": "f16", "params": {"tile_n": 64}, "ms": 2.0, "tflops": 1.0, "gbs": 1.0, "status": 0},
            {"shape": [64, 64, 64], "dtype": "f16", "params": {"tile_n": 16}, "ms": 1.0, "tflops": 2.0, "gbs": 2.0, "status": 0},
            {"shape": [64, 64, 64], "dtype": "f16", "params": {"tile_n": 32}, "ms": 0.5, "tflops": 4.0, "gbs": 4.0, "status": 5},
            {"shape": [128, 64, 64], "dtype": "f16", "params": {"tile_n": 8}, "ms": 0.1, "tflops": 9.0, "gbs": 9.0, "status": 0}]
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    assert len(t.load(path)) == 4
    assert t.best(path, 64, 64, 64) == {"tile_n": 16}            # fastest with a clean device status
    assert t.best(path, 64, 64, 64, "bf16") is None
    assert t.best(str(tmp_path / "missing.jsonl"), 64, 64, 64) is None


def test_timeline_summary_of_stamps():
    """cuda-kernel-opt_b200/timeline.py: per-milestone mean / min / max over the CTAs that had work, measured
    from the first CTA's entry; CTAs that never entered or never saw an accumulator are left out, and so are
    milestones nobody stamped."""
    import numpy as np
    from __graft_entry__ import load_package
    load_package()
    tl = importlib.import_module("cuda_kernel_opt_b200.timeline")
    stamps = np.zeros((4, 32), np.int64)
    base = 1_000_000
    stamps[0, 13], stamps[0, 14], stamps[0, 22], stamps[0, 15] = base, base + 500, base + 4000, base + 9000
    stamps[1, 13], stamps[1, 14], stamps[1, 22], stamps[1, 15] = base + 100, base + 700, base + 5000, base + 9500
    stamps[2, 13], stamps[2, 14], stamps[2, 15] = base + 50, base + 600, base + 800          # entered, no work
    entered, working, rows = tl.summarise(stamps)                                               # CTA 3 never entered
    assert (entered, working) == (3, 2)
    got = {name: (mean, lo, hi) for name, mean, lo, hi in rows}
    assert got["kernel entry"] == (50.0, 0, 100)
    assert got["set-up barrier passed"] == (600.0, 500, 700)
    assert got["epilogue: first accumulator ready"] == (4500.0, 4000, 5000)
    assert got["exit"] == (9250.0, 9000, 9500)
    assert "mma: first stage full" not in got
    assert [name for name, *_ in rows] == [n for _, n in tl.MILESTONES if n in got]             # milestone order kept
    assert tl.summarise(np.zeros((2, 32), np.int64)) == (0, 0, [])
