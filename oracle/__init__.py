"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE, never a product path).

Only tests, the smoke check and the bench's CPU-baseline legs import this package. It wraps

* ``liboracle.so``  - gemm_oracle.c, the restatement of the reference's host check
  (matmul_test.h:294-298, :316-320) plus an independent copy of the seeded input generator;
* ``_ref/libref_matmul.so`` - the reference's own ``MatmulTestGemmSquare`` compiled from the
  reference tree (ref_driver.cpp); present only where ``make -C oracle`` found that tree.

Arrays are numpy; fp16/bf16 operands travel as ``uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")
_REF = os.path.join(_HERE, "_ref", "libref_matmul.so")

FP16, BF16 = 0, 1
UNIFORM, NORMAL = 0, 1
# tensor ids of the generator: which operand an index stream belongs to
TENSOR_A, TENSOR_B, TENSOR_C = 1, 2, 3


def build(force: bool = False) -> None:
    """Compile liboracle.so (and _ref when the reference tree is present) with oracle/Makefile."""
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(
            os.path.join(_HERE, "gemm_oracle.c")):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    # the reference checkout: named by REFERENCE_TREE, else looked for beside this repository
    ref_tree = os.environ.get("REFERENCE_TREE") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    if os.path.exists(os.path.join(ref_tree, "matmul_test.h")) and (force or not os.path.exists(_REF)):
        subprocess.run(["make", "-C", _HERE, "ref", f"REFERENCE={ref_tree}"], check=True, capture_output=True)


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB)
        i64, f32, u64, vp = C.c_int64, C.c_float, C.c_uint64, C.c_void_p
        L.oracle_gemm.argtypes = [vp, vp, vp, vp, f32, f32, i64, i64, i64, C.c_int, C.c_int]
        L.oracle_gemm.restype = C.c_int
        L.oracle_gemm_rows.argtypes = [vp, vp, vp, vp, f32, f32, i64, i64, i64, C.c_int, i64, i64, C.c_int]
        L.oracle_gemm_rows.restype = C.c_int
        L.oracle_gemm_scalar.argtypes = [vp, vp, vp, vp, f32, f32, i64, i64, i64, C.c_int]
        L.oracle_gemm_scalar.restype = None
        L.oracle_gemm_elements.argtypes = [vp, vp, vp, f32, f32, i64, i64, C.c_int, vp, i64, vp, vp]
        L.oracle_gemm_elements.restype = None
        L.oracle_count_incorrect.argtypes = [vp, vp, i64, f32]
        L.oracle_count_incorrect.restype = i64
        L.oracle_constant_expected.argtypes = [f32, f32, f32, f32, f32, i64]
        L.oracle_constant_expected.restype = f32
        L.oracle_fill_u16.argtypes = [vp, i64, i64, u64, u64, C.c_int, f32, C.c_int]
        L.oracle_fill_u16.restype = None
        L.oracle_fill_f32.argtypes = [vp, i64, i64, u64, u64, C.c_int, f32]
        L.oracle_fill_f32.restype = None
        L.oracle_to_float.argtypes = [vp, vp, i64, C.c_int]
        L.oracle_to_float.restype = None
        L.oracle_max_threads.restype = C.c_int
        _lib = L
    return _lib


def have_ref() -> bool:
    return os.path.exists(_REF)


def ref():
    global _ref
    if _ref is None:
        R = C.CDLL(_REF)
        vp, f32 = C.c_void_p, C.c_float
        R.ref_create.argtypes = [C.c_int, C.c_int]
        R.ref_create.restype = vp
        R.ref_destroy.argtypes = [vp, C.c_int]
        R.ref_destroy.restype = None
        R.ref_load.argtypes = [vp, C.c_int, vp, vp, vp, C.c_int]
        R.ref_load.restype = C.c_int
        R.ref_count_incorrect.argtypes = [vp, C.c_int, vp, C.c_int, f32, f32, f32]
        R.ref_count_incorrect.restype = C.c_int
        R.ref_constant_is_correct.argtypes = [vp, C.c_int, f32, f32, f32]
        R.ref_constant_is_correct.restype = C.c_int
        if hasattr(R, "ref_half_count_incorrect"):
            R.ref_half_count_incorrect.argtypes = [C.c_int, vp, vp, vp, vp, C.c_int, f32, f32, f32]
            R.ref_half_count_incorrect.restype = C.c_int
        _ref = R
    return _ref


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _chk(a, dtype, name):
    assert a.dtype == dtype and a.flags["C_CONTIGUOUS"], f"{name}: need contiguous {dtype}"
    return a


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def gemm(A, Bt, Cm=None, alpha=1.0, beta=0.0, dtype=FP16, threads=0, rows=None, scalar=False):
    """D = alpha*A*Bt^T + beta*C in the reference's arithmetic. A: (m,k) uint16, Bt: (n,k) uint16,
    Cm: (m,n) float32 or None. ``rows=(r0,r1)`` computes only that row range (others left 0)."""
    _chk(A, np.uint16, "A"); _chk(Bt, np.uint16, "Bt")
    m, k = A.shape
    n, k2 = Bt.shape
    assert k == k2
    if Cm is not None:
        _chk(Cm, np.float32, "C"); assert Cm.shape == (m, n)
    D = np.zeros((m, n), np.float32)
    if scalar:
        lib().oracle_gemm_scalar(_p(A), _p(Bt), _p(Cm), _p(D), alpha, beta, m, n, k, dtype)
        return D
    r0, r1 = (0, m) if rows is None else rows
    rc = lib().oracle_gemm_rows(_p(A), _p(Bt), _p(Cm), _p(D), alpha, beta, m, n, k, dtype, r0, r1, threads)
    if rc != 0:
        raise MemoryError("oracle_gemm_rows")
    return D


def gemm_elements(A, Bt, Cm, alpha, beta, idx, dtype=FP16):
    """Scattered elements (linear indices i*n+j): returns (fp32 in reference order, fp64)."""
    _chk(A, np.uint16, "A"); _chk(Bt, np.uint16, "Bt")
    n, k = Bt.shape
    idx = np.ascontiguousarray(idx, np.int64)
    o32 = np.empty(idx.shape, np.float32)
    o64 = np.empty(idx.shape, np.float64)
    lib().oracle_gemm_elements(_p(A), _p(Bt), _p(Cm), alpha, beta, n, k, dtype, _p(idx), idx.size, _p(o32), _p(o64))
    return o32, o64


def count_incorrect(expected, got, atol) -> int:
    e = np.ascontiguousarray(expected, np.float32); g = np.ascontiguousarray(got, np.float32)
    assert e.shape == g.shape
    return int(lib().oracle_count_incorrect(_p(e), _p(g), e.size, atol))


def constant_expected(a, b, c, alpha, beta, k) -> float:
    return float(lib().oracle_constant_expected(a, b, c, alpha, beta, k))


def fill_u16(shape, seed, tensor_id, dist=UNIFORM, sigma=1.0, dtype=FP16, begin=0):
    out = np.empty(shape, np.uint16)
    lib().oracle_fill_u16(_p(out), begin, out.size, seed, tensor_id, dist, sigma, dtype)
    return out


def fill_f32(shape, seed, tensor_id, dist=UNIFORM, sigma=1.0, begin=0):
    out = np.empty(shape, np.float32)
    lib().oracle_fill_f32(_p(out), begin, out.size, seed, tensor_id, dist, sigma)
    return out


def to_float(bits, dtype=FP16):
    bits = np.ascontiguousarray(bits, np.uint16)
    out = np.empty(bits.shape, np.float32)
    lib().oracle_to_float(_p(bits), _p(out), bits.size, dtype)
    return out


class RefSession:
    """The reference's MatmulTestGemmSquare holding an n x n problem (n == k)."""

    def __init__(self, n: int, dtype: int = FP16):
        self.n, self.dtype = n, dtype
        self.h = ref().ref_create(n, dtype)
        if not self.h:
            raise MemoryError("ref_create")

    def load(self, A, Bt, Cm=None):
        _chk(A, np.uint16, "A"); _chk(Bt, np.uint16, "Bt")
        assert Bt.shape == (self.n, self.n) and A.shape[1] == self.n
        self.m = A.shape[0]
        if Cm is not None:
            _chk(Cm, np.float32, "C")
        rc = ref().ref_load(self.h, self.dtype, _p(A), _p(Bt), _p(Cm), self.m)
        assert rc == 0

    def count_incorrect(self, res, alpha=1.0, beta=0.0, atol=0.0) -> int:
        res = np.ascontiguousarray(res, np.float32)
        assert res.shape == (self.m, self.n)
        return int(ref().ref_count_incorrect(self.h, self.dtype, _p(res), self.m, alpha, beta, atol))

    def close(self):
        if self.h:
            ref().ref_destroy(self.h, self.dtype)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def ref_constant_is_correct(res, alpha, beta, atol) -> bool:
    res = np.ascontiguousarray(res, np.float32)
    n = res.shape[0]
    assert res.shape == (n, n)
    return bool(ref().ref_constant_is_correct(_p(res), n, alpha, beta, atol))


def ref_half_count_incorrect(A, Bt, C16, res16, alpha, beta, atol) -> int:
    """The reference's <half, half> check (accumulation in half): how many elements of the fp16 result res16
    are off by more than atol. A: (m, n), Bt: (n, n), C16 / res16: (m, n) fp16 bit patterns (uint16)."""
    _chk(A, np.uint16, "A"); _chk(Bt, np.uint16, "Bt"); _chk(res16, np.uint16, "res")
    n = Bt.shape[0]
    assert Bt.shape == (n, n) and A.shape[1] == n and res16.shape == A.shape[:1] + (n,)
    if C16 is not None:
        _chk(C16, np.uint16, "C")
    return int(ref().ref_half_count_incorrect(n, _p(A), _p(Bt), _p(C16), _p(res16), A.shape[0], alpha, beta, atol))
