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


class Guarded:
    """A device tensor carved out of the middle of a larger allocation whose two margins ("guard bands")
    hold the byte 0xA5. A store that lands outside the tensor - a clipped edge that is off by a row, a
    transposed or swapped drain with the wrong pitch - changes a band instead of a neighbouring
    allocation nobody looks at; check() asserts both bands are untouched. Stands in for a memory
    checker on machines where none can be run. The tensor starts 512-byte aligned."""

    BYTE = 0xA5

    def __init__(self, torch, shape, dtype, fill=float("nan"), band_bytes=None):
        self.torch = torch
        elem = torch.empty((), dtype=dtype).element_size()
        numel = 1
        for d in shape:
            numel *= int(d)
        if band_bytes is None:          # at least 130 rows of the tensor (more than one tile row off) + 4 KiB
            row = int(shape[-1]) * elem if len(shape) > 1 else 0
            band_bytes = min(16 << 20, 130 * row + 4096)
        self.band = -(-band_bytes // 512) * 512
        self.nbytes = numel * elem
        self.buf = torch.full((2 * self.band + -(-self.nbytes // 512) * 512,), self.BYTE, dtype=torch.uint8, device="cuda")
        self.t = self.buf[self.band:self.band + self.nbytes].view(dtype).view(*shape)
        if fill is not None:
            self.t.fill_(fill)

    def check(self, what=""):
        lo = self.buf[:self.band]
        hi = self.buf[self.band + self.nbytes:]
        bad_lo = int((lo != self.BYTE).sum())
        bad_hi = int((hi != self.BYTE).sum())
        assert bad_lo == 0 and bad_hi == 0, (f"{what}: {bad_lo} bytes changed before the tensor, {bad_hi} after it "
                                             f"(first after: {int((hi != self.BYTE).nonzero()[0]) if bad_hi else None})")
