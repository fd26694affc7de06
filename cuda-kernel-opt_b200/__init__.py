"""Python face of libb200gemm.so, the B200 (sm_100a) asynchronous tensor-core GEMM.

The product is the C-ABI shared library (include/b200_gemm.h); this module only binds it with
ctypes so that Python harnesses (tests, bench) can call it with device pointers taken from torch
tensors. There is no CPU or PyTorch fallback: if the library is missing the import fails, and on
a machine without an sm_100 GPU every compute call raises ``B200Error``.

The directory name contains a hyphen, so import it through ``__graft_entry__.load_package()``
(which registers it as ``cuda_kernel_opt_b200``).
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, asdict

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("B200_GEMM_LIB") or os.path.join(_HERE, "libb200gemm.so")

OK, INVALID_CONFIG, INVALID_SHAPE, INVALID_POINTER, CUDA_ERROR, DEVICE_TIMEOUT, WORKSPACE_TOO_SMALL, UNSUPPORTED_DEVICE = range(8)
F16, BF16 = 0, 1
UNIFORM, NORMAL = 0, 1
TENSOR_A, TENSOR_B, TENSOR_C = 1, 2, 3

# every symbol include/b200_gemm.h declares
EXPORTS = [
    "b200_gemm_default_params", "b200_gemm_default_params_plain", "b200_gemm_default_params_for_call", "b200_gemm_validate", "b200_gemm_smem_bytes", "b200_gemm_workspace_bytes", "b200_gemm_schedule",
    "b200_gemm_f16", "b200_gemm_bf16", "b200_gemm_f16_out_f16", "b200_gemm_splitk_noalloc", "b200_gemm_push", "b200_push_reduce",
    "b200_peer_alloc", "b200_peer_free", "b200_peer_export", "b200_peer_import", "b200_peer_release", "b200_session_create", "b200_session_destroy", "b200_session_gemm_host", "b200_session_buffers", "b200_session_gemm_host_sharded",
    "b200_device_status", "b200_set_wait_budget_ns", "b200_set_profile_buffer", "b200_profile_slots", "b200_status_string", "b200_last_cuda_error", "b200_num_sms",
    "b200_fill_u16_device", "b200_fill_f32_device", "b200_fill_u16_host", "b200_fill_f32_host",
]


class Params(C.Structure):
    """struct b200_gemm_params."""
    _fields_ = [(n, C.c_int) for n in (
        "tile_m", "tile_n", "segment_dim_k", "bar_steps_a", "bar_steps_b", "bar_step_rows_a", "bar_step_rows_b",
        "tile_group_m", "num_stages", "num_producer_warps", "num_consumer_warps", "num_sms", "cta_group", "split_k",
        "epilogue", "l2_hint", "diagnostic", "k_order", "tail_split", "swap_ab", "cluster_reduce", "overlap_launch")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_ if n != "reserved"}


class B200Error(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: status {status} ({status_string(status)}), cuda error {lib().b200_last_cuda_error()}")


_lib = None


def lib():
    """The loaded shared library. Raises OSError if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} is missing: build it with cuda-kernel-opt_b200/build.py (there is no fallback path)")
        L = C.CDLL(LIB_PATH)
        i64, f32, u64, vp, sz = C.c_int64, C.c_float, C.c_uint64, C.c_void_p, C.c_size_t
        PP = C.POINTER(Params)
        L.b200_gemm_default_params.argtypes = [i64, i64, i64, C.c_int, PP]
        L.b200_gemm_default_params_plain.argtypes = [i64, i64, i64, C.c_int, PP]
        L.b200_gemm_default_params_for_call.argtypes = [i64, i64, i64, C.c_int, C.c_float, C.c_int, PP]
        L.b200_gemm_default_params_for_call.restype = C.c_int
        L.b200_gemm_validate.argtypes = [i64, i64, i64, C.c_int, PP]
        L.b200_gemm_smem_bytes.argtypes = [C.c_int, PP]
        L.b200_gemm_smem_bytes.restype = i64
        L.b200_gemm_workspace_bytes.argtypes = [i64, i64, i64, PP]
        L.b200_gemm_workspace_bytes.restype = i64
        L.b200_gemm_schedule.argtypes = [i64, i64, i64, PP, C.c_int, C.c_int, C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int)]
        L.b200_gemm_schedule.restype = C.c_int
        for fn in (L.b200_gemm_f16, L.b200_gemm_bf16):
            fn.argtypes = [vp, vp, vp, vp, f32, f32, i64, i64, i64, PP, vp, sz, vp]
            fn.restype = C.c_int
        L.b200_gemm_f16_out_f16.argtypes = [vp, vp, vp, vp, f32, f32, i64, i64, i64, PP, vp]
        L.b200_gemm_f16_out_f16.restype = C.c_int
        L.b200_gemm_splitk_noalloc.argtypes = [C.c_int, vp, vp, vp, vp, f32, f32, i64, i64, i64, PP, vp]
        L.b200_gemm_splitk_noalloc.restype = C.c_int
        L.b200_gemm_push.argtypes = [C.c_int, vp, vp, i64, i64, i64, PP, C.c_int, C.c_int, C.POINTER(vp), C.POINTER(vp), vp, C.c_int, vp, sz, vp]
        L.b200_push_reduce.argtypes = [vp, vp, C.c_int, C.c_int, vp, vp, f32, f32, i64, i64, vp]
        L.b200_peer_alloc.argtypes = [sz, C.POINTER(vp)]
        L.b200_peer_free.argtypes = [vp]
        L.b200_peer_export.argtypes = [vp, C.c_char_p]
        L.b200_peer_import.argtypes = [C.c_char_p, C.POINTER(vp)]
        L.b200_peer_release.argtypes = [vp]
        L.b200_session_create.argtypes = [i64, i64, i64, C.POINTER(vp)]
        L.b200_session_destroy.argtypes = [vp]
        L.b200_session_destroy.restype = None
        L.b200_session_gemm_host.argtypes = [vp, C.c_int, vp, vp, vp, vp, f32, f32, i64, i64, i64, PP]
        L.b200_session_buffers.argtypes = [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]
        L.b200_session_gemm_host_sharded.argtypes = [vp, C.c_int, vp, vp, vp, vp, f32, f32, i64, i64, i64, C.c_int, C.c_int,
                                                     C.POINTER(vp), C.POINTER(vp), C.c_int, PP]
        L.b200_device_status.argtypes = [vp, C.POINTER(C.c_int * 4)]
        L.b200_set_wait_budget_ns.argtypes = [u64]
        L.b200_set_wait_budget_ns.restype = None
        L.b200_set_profile_buffer.argtypes = [vp, C.c_int]
        L.b200_set_profile_buffer.restype = None
        L.b200_profile_slots.argtypes = []
        L.b200_profile_slots.restype = C.c_int
        L.b200_status_string.argtypes = [C.c_int]
        L.b200_status_string.restype = C.c_char_p
        L.b200_fill_u16_device.argtypes = [vp, i64, i64, u64, u64, C.c_int, f32, C.c_int, vp]
        L.b200_fill_f32_device.argtypes = [vp, i64, i64, u64, u64, C.c_int, f32, vp]
        L.b200_fill_u16_host.argtypes = [vp, i64, i64, u64, u64, C.c_int, f32, C.c_int]
        L.b200_fill_u16_host.restype = None
        L.b200_fill_f32_host.argtypes = [vp, i64, i64, u64, u64, C.c_int, f32]
        L.b200_fill_f32_host.restype = None
        _lib = L
    return _lib


def status_string(status: int) -> str:
    return lib().b200_status_string(status).decode()


def default_params(M: int, N: int, K: int, dtype: int = F16, **overrides) -> Params:
    """b200_gemm_default_params plus keyword overrides of single tunables.

    Overriding the tile (tile_m / tile_n / cta_group) starts from the one-CTA defaults unless the
    override itself asks for the two-CTA pair, so that a partial override stays a valid whole."""
    p = Params()
    tile_keys = {"tile_m", "tile_n", "cta_group"} & set(overrides)
    want_pair = (overrides.get("cta_group", 0) == 2 or overrides.get("tile_m", 0) == 256) and not overrides.get("swap_ab")
    want_swap = overrides.get("swap_ab")
    if want_swap is None and (tile_keys or overrides.get("tail_split") or overrides.get("epilogue")):
        want_swap = 0          # tile_m / tile_n change meaning with swap_ab: an override names the plain form
    base_m = M if (not tile_keys or want_pair) else min(M, 128)
    fn = lib().b200_gemm_default_params_plain if want_swap == 0 else lib().b200_gemm_default_params
    st = fn(base_m, N, K, dtype, C.byref(p))
    if st != OK:
        raise B200Error(st, "b200_gemm_default_params")
    if tile_keys and not want_pair and M > 128:
        p.l2_hint = 0          # the skinny-shape hint of the reduced-M base does not apply
    if want_pair and p.cta_group != 2:
        p.tile_m, p.tile_n, p.cta_group, p.num_stages, p.l2_hint = 256, 256, 2, 6, 3
    if want_swap == 1 and (not p.swap_ab or overrides.get("cta_group", p.cta_group) != p.cta_group):
        pair_swap = overrides.get("cta_group", 0) == 2     # swapped pair: 256 weight rows per tile, tile_m a multiple of 32
        gran = 32 if pair_swap else 16
        p.swap_ab, p.tile_m, p.tile_n = 1, min(256, -(-M // gran) * gran), 256 if pair_swap else 128
        p.cta_group, p.epilogue, p.segment_dim_k = 2 if pair_swap else 1, 0, 64
        p.num_stages, p.num_producer_warps = 8, 1
        p.split_k, p.cluster_reduce = 1, 0
    for k, v in overrides.items():
        if not hasattr(p, k):
            raise AttributeError(k)
        setattr(p, k, v)
    if "split_k" in overrides and "cluster_reduce" not in overrides and p.cluster_reduce and p.split_k not in (2, 4, 8):
        p.cluster_reduce = 0            # not a cluster size: the slices meet in the workspace
    # keep "shift off" consistent when only the tile was overridden
    if "bar_step_rows_b" not in overrides:
        p.bar_step_rows_b = p.tile_n
    if "bar_step_rows_a" not in overrides:
        p.bar_step_rows_a = p.tile_m
    if "epilogue" not in overrides and lib().b200_gemm_smem_bytes(dtype, C.byref(p)) < 0 and "num_stages" in overrides:
        p.epilogue = 0                  # an explicit depth wins over the default TMA-store staging
    if "num_stages" not in overrides:   # a default depth chosen for another tile may not fit this one
        while p.num_stages > 1 and lib().b200_gemm_smem_bytes(dtype, C.byref(p)) < 0:
            p.num_stages -= 1
    return p


def validate(M, N, K, dtype, p: Params) -> int:
    return lib().b200_gemm_validate(M, N, K, dtype, C.byref(p))


def smem_bytes(dtype, p: Params) -> int:
    return lib().b200_gemm_smem_bytes(dtype, C.byref(p))


def workspace_bytes(M, N, K, p: Params) -> int:
    return lib().b200_gemm_workspace_bytes(M, N, K, C.byref(p))


def schedule(M, N, K, p: Params, num_sms: int = 148, group: int = 0):
    """b200_gemm_schedule: (number of CTA groups, [(m0, n0, seg_begin, seg_end, kind, slice), ...]) for one group.
    Host arithmetic only. Raises ValueError for an invalid configuration or group."""
    groups = C.c_int(0)
    n = lib().b200_gemm_schedule(M, N, K, C.byref(p), num_sms, group, None, 0, C.byref(groups))
    if n < 0:
        raise ValueError("invalid configuration or group")
    buf = (C.c_int * (6 * max(n, 1)))()
    lib().b200_gemm_schedule(M, N, K, C.byref(p), num_sms, group, buf, n, None)
    return groups.value, [tuple(buf[6 * i:6 * i + 6]) for i in range(n)]


def gemm_raw(dtype, A_ptr, Bt_ptr, C_ptr, D_ptr, alpha, beta, M, N, K, p, ws_ptr=None, ws_bytes=0, stream=None) -> int:
    """Direct call of b200_gemm_f16 / b200_gemm_bf16 with raw device addresses. Returns the status."""
    fn = lib().b200_gemm_bf16 if dtype == BF16 else lib().b200_gemm_f16
    return fn(A_ptr, Bt_ptr, C_ptr, D_ptr, alpha, beta, M, N, K, C.byref(p) if p is not None else None, ws_ptr, ws_bytes, stream)


def gemm_splitk_noalloc_raw(dtype, A_ptr, Bt_ptr, C_ptr, D_ptr, alpha, beta, M, N, K, p, stream=None) -> int:
    """Direct call of b200_gemm_splitk_noalloc (split-K with the library's built-in scratch:
    no allocation, no caller workspace; split_k * M * N <= 8 Mi). Returns the status."""
    return lib().b200_gemm_splitk_noalloc(dtype, A_ptr, Bt_ptr, C_ptr, D_ptr, alpha, beta, M, N, K, C.byref(p), stream)


def gemm(A, Bt, Cm=None, D=None, alpha=1.0, beta=0.0, params: Params | None = None, workspace=None, stream=None):
    """D = alpha * A @ Bt.T + beta * C on torch CUDA tensors (fp16 or bf16 A, Bt; fp32 C, D).

    Thin convenience over the C ABI: it takes addresses from the tensors, allocates D (and the
    split-K workspace) with torch when not given, and raises B200Error on a non-zero status."""
    import torch
    assert A.is_cuda and Bt.is_cuda and A.is_contiguous() and Bt.is_contiguous()
    assert A.dtype == Bt.dtype and A.dtype in (torch.float16, torch.bfloat16)
    M, K = A.shape
    N, K2 = Bt.shape
    assert K == K2
    dtype = BF16 if A.dtype == torch.bfloat16 else F16
    if D is None:
        D = torch.empty((M, N), dtype=torch.float32, device=A.device)
    assert D.dtype in (torch.float32, torch.float16) and D.is_contiguous() and D.shape == (M, N)
    if Cm is not None:
        assert Cm.dtype == D.dtype and Cm.is_contiguous() and Cm.shape == (M, N)
    if params is not None:
        p = params
    else:
        # the defaults of this call: the library keeps large squares off the tall pair when there is a C to read or D is fp16
        p = Params()
        st = lib().b200_gemm_default_params_for_call(M, N, K, dtype, float(beta), 1 if D.dtype == torch.float16 else 0, C.byref(p))
        if st != OK:
            raise B200Error(st, "b200_gemm_default_params_for_call")
    if D.dtype == torch.float16:
        # fp16 C and D (the reference's DT = DT_ACC = half instances): b200_gemm_f16_out_f16, no workspace forms
        assert dtype == F16, "fp16 output goes with fp16 operands"
        sptr = stream if stream is not None else torch.cuda.current_stream(A.device).cuda_stream
        with torch.cuda.device(A.device):
            # no tunables given: the library picks (it keeps large squares off the tall pair here, whose exposed drain only
            # pays with the TMA-store epilogue that fp16 output does not have)
            st = lib().b200_gemm_f16_out_f16(A.data_ptr(), Bt.data_ptr(), Cm.data_ptr() if Cm is not None else None, D.data_ptr(),
                                             alpha, beta, M, N, K, C.byref(p), sptr)
        if st != OK:
            raise B200Error(st, "b200_gemm_f16_out_f16")
        return D
    need = workspace_bytes(M, N, K, p)
    if need and workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=A.device)
    sptr = stream if stream is not None else torch.cuda.current_stream(A.device).cuda_stream
    with torch.cuda.device(A.device):
        st = gemm_raw(dtype, A.data_ptr(), Bt.data_ptr(), Cm.data_ptr() if Cm is not None else None, D.data_ptr(),
                      alpha, beta, M, N, K, p, workspace.data_ptr() if workspace is not None else None,
                      workspace.numel() * workspace.element_size() if workspace is not None else 0, sptr)
    if st != OK:
        raise B200Error(st, "b200_gemm")
    return D


def device_status(stream=None):
    """Synchronises and returns (status, [code, block, barrier, phase]) of the bounded-wait record."""
    info = (C.c_int * 4)()
    st = lib().b200_device_status(stream, C.byref(info))
    return st, list(info)


def set_wait_budget_ns(ns: int) -> None:
    lib().b200_set_wait_budget_ns(ns)


def profile_slots() -> int:
    """int64 slots per CTA of the profile buffer (16; 32 in a -DB200_TIMELINE build)."""
    return lib().b200_profile_slots()


def num_sms() -> int:
    return lib().b200_num_sms()


class Session:
    """b200_session: device buffers at maximal dimensions + the host-buffer GEMM call."""

    def __init__(self, max_m, max_n, max_k):
        self.h = C.c_void_p()
        st = lib().b200_session_create(max_m, max_n, max_k, C.byref(self.h))
        if st != OK:
            raise B200Error(st, "b200_session_create")

    def gemm_host(self, dtype, hA, hBt, hC, hD, alpha, beta, M, N, K, params=None):
        """hA, hBt, hC, hD: objects with a host address: numpy arrays or (pinned) torch CPU tensors."""
        def addr(x):
            if x is None:
                return None
            return x.data_ptr() if hasattr(x, "data_ptr") else x.ctypes.data
        st = lib().b200_session_gemm_host(self.h, dtype, addr(hA), addr(hBt), addr(hC), addr(hD), alpha, beta, M, N, K,
                                          C.byref(params) if params is not None else None)
        if st != OK:
            raise B200Error(st, "b200_session_gemm_host")

    def close(self):
        if self.h:
            lib().b200_session_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def fill_u16_host(shape, seed, tensor_id, dist=UNIFORM, sigma=1.0, dtype=F16, begin=0):
    import numpy as np
    out = np.empty(shape, np.uint16)
    lib().b200_fill_u16_host(out.ctypes.data, begin, out.size, seed, tensor_id, dist, sigma, dtype)
    return out


def fill_f32_host(shape, seed, tensor_id, dist=UNIFORM, sigma=1.0, begin=0):
    import numpy as np
    out = np.empty(shape, np.float32)
    lib().b200_fill_f32_host(out.ctypes.data, begin, out.size, seed, tensor_id, dist, sigma)
    return out


def fill_device(t, seed, tensor_id, dist=UNIFORM, sigma=1.0, begin=0):
    """Fills a contiguous torch CUDA tensor (fp16, bf16 or fp32) in place from the seeded generator."""
    import torch
    assert t.is_cuda and t.is_contiguous()
    sptr = torch.cuda.current_stream(t.device).cuda_stream
    with torch.cuda.device(t.device):
        if t.dtype == torch.float32:
            st = lib().b200_fill_f32_device(t.data_ptr(), begin, t.numel(), seed, tensor_id, dist, sigma, sptr)
        else:
            assert t.dtype in (torch.float16, torch.bfloat16)
            st = lib().b200_fill_u16_device(t.data_ptr(), begin, t.numel(), seed, tensor_id, dist, sigma,
                                            BF16 if t.dtype == torch.bfloat16 else F16, sptr)
    if st != OK:
        raise B200Error(st, "b200_fill_device")
    return t
