"""Generates tests/golden/*.npz: seeded inputs -> outputs of the CPU oracle, each checked at
generation time against the REFERENCE's own host check compiled from its tree.

Run where the reference tree is present (``python tests/golden/make_golden.py`` from the repo
root, after ``make -C oracle``). For every case with n == k the oracle's result D is handed to
the reference's ``MatmulTestGemmSquare::GetNumIncorrect`` (matmul_test.h:307-326) with atol = 0;
the case is written only if the count is 0, i.e. D equals the reference's recompute in every bit
that its comparison can see. Cases with n != k cannot be given to the reference (it reads B^T
with pitch n, matmul_test.h:318) and are marked ``ref_checked = 0``.

The fixtures carry the outputs only; inputs are regenerated from (seed, tensor id) by the
generator, whose own known answers are stored in ``generator_kat.npz``.
"""
import hashlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# name, dtype, m, n, k, seed, alpha, beta, dist_a (dist, sigma), dist_b
CASES = [
    ("f16_64", oracle.FP16, 64, 64, 64, 10, 1.0, 1.0, (0, 1.0), (0, 1.0)),
    ("f16_128", oracle.FP16, 128, 128, 128, 11, 1.0, 1.0, (0, 1.0), (0, 1.0)),
    ("f16_256_ab", oracle.FP16, 256, 256, 256, 12, 1.5, -0.5, (0, 1.0), (0, 1.0)),
    ("f16_slab_128x256", oracle.FP16, 128, 256, 256, 13, 1.0, 0.0, (0, 1.0), (0, 1.0)),
    ("bf16_128", oracle.BF16, 128, 128, 128, 14, 1.0, 1.0, (0, 1.0), (0, 1.0)),
    ("bf16_256_normal", oracle.BF16, 128, 256, 256, 15, 1.0, 0.0, (1, 1.0), (1, 0.02)),
    ("f16_rect_128x192x320", oracle.FP16, 128, 192, 320, 16, 1.0, 1.0, (0, 1.0), (0, 1.0)),
    ("bf16_rect_16x256x512", oracle.BF16, 16, 256, 512, 17, 1.0, 0.0, (1, 1.0), (1, 0.02)),
]


def inputs(dtype, m, n, k, seed, da, db):
    A = oracle.fill_u16((m, k), seed, oracle.TENSOR_A, da[0], da[1], dtype)
    Bt = oracle.fill_u16((n, k), seed, oracle.TENSOR_B, db[0], db[1], dtype)
    Cm = oracle.fill_f32((m, n), seed, oracle.TENSOR_C)
    return A, Bt, Cm


def main():
    assert oracle.have_ref(), "build oracle/_ref first (make -C oracle) where the reference tree is present"
    for name, dtype, m, n, k, seed, alpha, beta, da, db in CASES:
        A, Bt, Cm = inputs(dtype, m, n, k, seed, da, db)
        D = oracle.gemm(A, Bt, Cm, alpha, beta, dtype)
        assert (D == oracle.gemm(A, Bt, Cm, alpha, beta, dtype, scalar=True)).all()
        ref_checked = 0
        if n == k:
            s = oracle.RefSession(n, dtype)
            s.load(A, Bt, Cm)
            bad = s.count_incorrect(D, alpha, beta, 0.0)
            assert bad == 0, f"{name}: reference disagrees on {bad} elements"
            s.close()
            ref_checked = 1
        np.savez_compressed(os.path.join(HERE, name + ".npz"), D=D, dtype=dtype, m=m, n=n, k=k, seed=seed,
                            alpha=np.float32(alpha), beta=np.float32(beta), dist_a=np.array(da), dist_b=np.array(db),
                            ref_checked=ref_checked)
        print(f"{name}: ref_checked={ref_checked}")

    # Config 1 of the baseline: 1024^3 fp16 U[-1,1) seed 0, alpha=1, beta=0. 4 MiB of output is
    # kept as a digest plus a sample.
    A, Bt, _ = inputs(oracle.FP16, 1024, 1024, 1024, 0, (0, 1.0), (0, 1.0))
    D = oracle.gemm(A, Bt, None, 1.0, 0.0, oracle.FP16)
    s = oracle.RefSession(1024, oracle.FP16)
    s.load(A, Bt, None)
    assert s.count_incorrect(D, 1.0, 0.0, 0.0) == 0
    s.close()
    np.savez_compressed(os.path.join(HERE, "c1_1024_digest.npz"),
                        sha256=np.frombuffer(hashlib.sha256(D.tobytes()).digest(), np.uint8),
                        sample_idx=np.arange(0, 1024 * 1024, 4099, dtype=np.int64),
                        sample=D.reshape(-1)[::4099].copy(), ref_checked=1)
    print("c1_1024_digest: ref_checked=1")

    # Constant family (A = 1, B = 10, C = 1; matmul_test.h:227-232): closed form judged by the
    # reference's IsCorrect at its own atol of 1e-3.
    rows = []
    for kk in (64, 128, 512, 1024):
        for alpha, beta in ((1.0, 1.0), (2.0, 0.0)):
            v = oracle.constant_expected(1.0, 10.0, 1.0, alpha, beta, kk)
            assert oracle.ref_constant_is_correct(np.full((kk, kk), v, np.float32), alpha, beta, 1e-3)
            rows.append((kk, alpha, beta, v))
    np.savez_compressed(os.path.join(HERE, "constant_family.npz"), rows=np.array(rows, np.float64))

    # Known answers of the generator itself.
    np.savez_compressed(
        os.path.join(HERE, "generator_kat.npz"),
        u_f16=oracle.fill_u16((64,), 0, oracle.TENSOR_A, 0, 1.0, oracle.FP16),
        u_bf16=oracle.fill_u16((64,), 2, oracle.TENSOR_B, 0, 1.0, oracle.BF16),
        n_bf16=oracle.fill_u16((64,), 3, oracle.TENSOR_B, 1, 0.02, oracle.BF16),
        u_f32=oracle.fill_f32((64,), 4, oracle.TENSOR_C),
        u_f16_offset=oracle.fill_u16((64,), 0, oracle.TENSOR_A, 0, 1.0, oracle.FP16, begin=1 << 33),
    )
    print("done")


if __name__ == "__main__":
    main()
