"""Shared pieces of the parity tests: seeded inputs, tolerance, upload."""
import numpy as np

GOLDEN = __import__("os").path.join(__import__("os").path.dirname(__import__("os").path.abspath(__file__)), "golden")


def inputs(gen, dtype, m, n, k, seed, dist_a=(0, 1.0), dist_b=(0, 1.0)):
    """A (m,k), Bt (n,k) as uint16 bit patterns and C (m,n) fp32 from the seeded generator `gen`
    (either the oracle module or the package: both expose fill_u16 / fill_f32 style functions)."""
    fill16 = getattr(gen, "fill_u16", None) or gen.fill_u16_host
    fill32 = getattr(gen, "fill_f32", None) or gen.fill_f32_host
    A = fill16((m, k), seed, 1, int(dist_a[0]), float(dist_a[1]), dtype)
    Bt = fill16((n, k), seed, 2, int(dist_b[0]), float(dist_b[1]), dtype)
    Cm = fill32((m, n), seed, 3)
    return A, Bt, Cm


def tolerance_ok(got, want, k, scale=1.0):
    """The stated bar: relative Frobenius error <= 1e-3 and per-element |err| <= 2^-10 * sqrt(K)
    (times `scale` = max|a| * max|b| for inputs outside [-1, 1])."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    if not np.isfinite(got).all():
        return False, "non-finite output"
    rel = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
    err = np.abs(got - want).max()
    bound = 2.0 ** -10 * np.sqrt(k) * scale
    return (rel <= 1e-3 and err <= bound), f"rel Frobenius {rel:.3e} (<= 1e-3), max|err| {err:.3e} (<= {bound:.3e})"


def to_device(torch, bits, dtype_code):
    t = torch.from_numpy(bits.view(np.int16)).cuda()
    return t.view(torch.bfloat16 if dtype_code == 1 else torch.float16)
