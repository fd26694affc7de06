"""How one GEMM is split over the GPUs of a box: one process per GPU, no data-path collective
unless K is split.

The reference is single-GPU (cudaSetDevice(0), matmul_shmem_tc_async_opt_port_2.cu:1503-1510);
output tiles are independent, so the split is by rows of A (and D), by rows of B^T (columns of D),
or by K with an fp32 reduce-scatter of the partial products.
"""
from __future__ import annotations

from dataclasses import dataclass


def _split(total: int, world: int, rank: int, align: int) -> tuple[int, int]:
    """Contiguous range of `total` for `rank`, boundaries on multiples of `align` (the last range
    takes what is left). Ranges cover [0, total) without overlap; a range may be empty."""
    if world < 1 or not (0 <= rank < world) or align < 1 or total < 0:
        raise ValueError("bad split arguments")
    units = (total + align - 1) // align
    lo = (units * rank) // world
    hi = (units * (rank + 1)) // world
    return min(lo * align, total), min(hi * align, total)


@dataclass(frozen=True)
class Shard:
    kind: str      # "m", "n" or "k"
    rank: int
    world: int
    begin: int
    end: int

    @property
    def size(self) -> int:
        return self.end - self.begin


def m_shard(M: int, world: int, rank: int, tile_m: int = 128) -> Shard:
    """Rows [begin, end) of A and D for this rank; B^T is replicated; no collective."""
    b, e = _split(M, world, rank, tile_m)
    return Shard("m", rank, world, b, e)


def n_shard(N: int, world: int, rank: int, tile_n: int = 256) -> Shard:
    """Rows [begin, end) of B^T (= columns of D) for this rank; A is replicated; the column
    blocks of D stay distributed; no collective."""
    b, e = _split(N, world, rank, tile_n)
    return Shard("n", rank, world, b, e)


def k_shard(K: int, world: int, rank: int, segment_dim_k: int = 64) -> Shard:
    """Columns [begin, end) of A and of B^T for this rank; every rank produces a full m x n fp32
    partial, combined by reduce_scatter_rows."""
    b, e = _split(K, world, rank, segment_dim_k)
    return Shard("k", rank, world, b, e)


def reduce_scatter_rows(partial, group=None):
    """Sum of the ranks' partial m x n products, scattered by rows: rank r keeps rows
    [r*m/world, (r+1)*m/world). One torch.distributed reduce-scatter (NCCL over NVLink on GPUs,
    gloo on CPU). m must be a multiple of the world size."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    m, n = partial.shape
    if m % world:
        raise ValueError("rows must divide by the world size")
    out = torch.empty((m // world, n), dtype=partial.dtype, device=partial.device)
    if world == 1:
        out.copy_(partial)
        return out
    if partial.is_cuda:
        dist.reduce_scatter_tensor(out, partial.contiguous(), op=dist.ReduceOp.SUM, group=group)
    else:  # gloo has no reduce_scatter: all-reduce, then keep the owned rows
        full = partial.clone()
        dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
        r = dist.get_rank(group)
        out.copy_(full[r * (m // world):(r + 1) * (m // world)])
    return out


class PushExchange:
    """Split-K over the GPUs of a box with the reduce-scatter fused into the GEMM epilogue
    (b200_gemm_push / b200_push_reduce): peers' fp32 tiles arrive in this GPU's slot area by plain
    NVLink stores while the GEMM is still running; what is left after the GEMM is a flag wait
    and one ordered sum of `world` local slabs. torch.distributed only carries the 64-byte IPC
    handles at set-up.

    Two slot areas alternate by step. No per-step barrier is needed: a rank starts the push of step
    e+2 (same area as step e) only after its own reduce of step e+1, which waited for every peer's
    flag of step e+1, which each peer raised (in stream order) after its reduce of step e. A rank whose host
    falls behind may therefore find a peer's flag already one epoch ahead when its own reduce looks: the
    reduce accepts any flag that has reached its epoch (the data of its epoch sits in the other area, intact).
    """

    def __init__(self, pkg, M: int, N: int, group=None):
        import ctypes as C
        import torch
        import torch.distributed as dist
        self.pkg, self.C, self.dist, self.group = pkg, C, dist, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if M % self.world or (M // self.world) % 128:
            raise ValueError("rows per GPU must be a multiple of 128")
        self.M, self.N, self.rows = M, N, M // self.world
        lib = pkg.lib()
        self.slots = C.c_void_p()
        self.flags = C.c_void_p()
        self.done = C.c_void_p()
        for ptr, nbytes in ((self.slots, 2 * self.world * self.rows * N * 4), (self.flags, 64 * 4), (self.done, 64)):
            st = lib.b200_peer_alloc(nbytes, C.byref(ptr))
            if st != pkg.OK:
                raise pkg.B200Error(st, "b200_peer_alloc")
        handles = []
        for ptr in (self.slots, self.flags):
            buf = C.create_string_buffer(64)
            st = lib.b200_peer_export(ptr, buf)
            if st != pkg.OK:
                raise pkg.B200Error(st, "b200_peer_export")
            handles.append(bytes(buf.raw))
        gathered = [None] * self.world
        dist.all_gather_object(gathered, handles, group=group)
        self.imported = []
        self.area_bytes = self.world * self.rows * N * 4
        self.slot_ptrs = (C.c_void_p * 8)()
        self.flag_ptrs = (C.c_void_p * 8)()
        for o in range(self.world):
            if o == self.rank:
                self.slot_ptrs[o], self.flag_ptrs[o] = self.slots.value, self.flags.value
                continue
            for which, arr in ((0, self.slot_ptrs), (1, self.flag_ptrs)):
                out = C.c_void_p()
                st = lib.b200_peer_import(gathered[o][which], C.byref(out))
                if st != pkg.OK:
                    raise pkg.B200Error(st, "b200_peer_import")
                arr[o] = out.value
                self.imported.append(out)
        self.slot_ptrs_odd = (C.c_void_p * 8)()
        for o in range(self.world):
            self.slot_ptrs_odd[o] = self.slot_ptrs[o] + self.area_bytes
        self.epoch = 0
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def push(self, A, Bt, params, stream=None, workspace=None):
        """First half of a step: this rank's K slice is multiplied and every finished tile is stored into
        its owner's slot area (b200_gemm_push). Starts a new epoch. Asynchronous on the current stream."""
        import torch
        pkg, lib = self.pkg, self.pkg.lib()
        dtype = pkg.BF16 if A.dtype == torch.bfloat16 else pkg.F16
        self.epoch += 1
        sptr = stream if stream is not None else torch.cuda.current_stream(A.device).cuda_stream
        odd = self.epoch & 1
        need = pkg.workspace_bytes(self.M, self.N, A.shape[1], params)
        if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
            workspace = self._ws = torch.empty(need, dtype=torch.uint8, device=A.device)
        st = lib.b200_gemm_push(dtype, A.data_ptr(), Bt.data_ptr(), self.M, self.N, A.shape[1], self.C.byref(params),
                                self.world, self.rank, self.slot_ptrs_odd if odd else self.slot_ptrs, self.flag_ptrs,
                                self.done, self.epoch, workspace.data_ptr() if need else None, need, sptr)
        if st != pkg.OK:
            raise pkg.B200Error(st, "b200_gemm_push")

    def reduce(self, D_rows, Cm_rows=None, alpha=1.0, beta=0.0, stream=None):
        """Second half: waits (on the device, bounded) until every source's flag has reached the current epoch,
        then sums the slots of this rank's rows into D_rows (b200_push_reduce)."""
        import torch
        pkg, lib = self.pkg, self.pkg.lib()
        sptr = stream if stream is not None else torch.cuda.current_stream(D_rows.device).cuda_stream
        odd = self.epoch & 1
        st = lib.b200_push_reduce(self.slots.value + (self.area_bytes if odd else 0), self.flags, self.world, self.epoch,
                                  Cm_rows.data_ptr() if Cm_rows is not None else None, D_rows.data_ptr(), alpha, beta,
                                  self.rows, self.N, sptr)
        if st != pkg.OK:
            raise pkg.B200Error(st, "b200_push_reduce")
        return D_rows

    def gemm_reduce_scatter(self, A, Bt, D_rows, params, Cm_rows=None, alpha=1.0, beta=0.0, stream=None, workspace=None):
        """A: M x K_local, Bt: N x K_local (this rank's K slice); D_rows: (M/world) x N fp32, this
        rank's rows of the full product. Asynchronous on the current stream."""
        self.push(A, Bt, params, stream=stream, workspace=workspace)
        return self.reduce(D_rows, Cm_rows, alpha, beta, stream=stream)

    def close(self):
        import torch
        torch.cuda.synchronize()
        self.dist.barrier(group=self.group)
        lib = self.pkg.lib()
        for p in self.imported:
            lib.b200_peer_release(p)
        self.imported = []
        self.dist.barrier(group=self.group)
        for p in (self.slots, self.flags, self.done):
            if p:
                lib.b200_peer_free(p)
        self.slots = self.flags = self.done = None


class HostGemmMShard:
    """The host-buffer GEMM of an M-sharded square problem on the GPUs of a box (b200_session_gemm_host_sharded):
    every rank passes its rows of A, its N / world rows of B^T and a buffer for its rows of D, all in (pinned) host
    memory. B^T crosses PCIe once: each rank uploads its own rows and copies them to the other GPUs over NVLink,
    and multiplies column block by column block as the blocks arrive. torch.distributed only carries the IPC
    handles at set-up."""

    def __init__(self, pkg, m_rows: int, N: int, K: int, group=None):
        import ctypes as C
        import torch
        import torch.distributed as dist
        self.pkg, self.C, self.dist, self.group = pkg, C, dist, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if N % self.world or (N // self.world) % 256:
            raise ValueError("columns per GPU must be a multiple of 256")
        self.m_rows, self.N, self.K = m_rows, N, K
        lib = pkg.lib()
        self.session = pkg.Session(m_rows, N, K)
        dB = C.c_void_p()
        st = lib.b200_session_buffers(self.session.h, None, C.byref(dB), None, None)
        if st != pkg.OK:
            raise pkg.B200Error(st, "b200_session_buffers")
        self.flags = C.c_void_p()
        st = lib.b200_peer_alloc(64 * 4, C.byref(self.flags))
        if st != pkg.OK:
            raise pkg.B200Error(st, "b200_peer_alloc")
        handles = []
        for ptr in (dB, self.flags):
            buf = C.create_string_buffer(64)
            st = lib.b200_peer_export(ptr, buf)
            if st != pkg.OK:
                raise pkg.B200Error(st, "b200_peer_export")
            handles.append(bytes(buf.raw))
        gathered = [None] * self.world
        dist.all_gather_object(gathered, handles, group=group)
        self.imported = []
        self.bt_ptrs = (C.c_void_p * 8)()
        self.flag_ptrs = (C.c_void_p * 8)()
        for o in range(self.world):
            if o == self.rank:
                self.bt_ptrs[o], self.flag_ptrs[o] = dB.value, self.flags.value
                continue
            for which, arr in ((0, self.bt_ptrs), (1, self.flag_ptrs)):
                out = C.c_void_p()
                st = lib.b200_peer_import(gathered[o][which], C.byref(out))
                if st != pkg.OK:
                    raise pkg.B200Error(st, "b200_peer_import")
                arr[o] = out.value
                self.imported.append(out)
        self.epoch = 0
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def gemm(self, dtype, hA_rows, hBt_rows, hC_rows, hD_rows, alpha=1.0, beta=0.0, params=None):
        """hA_rows: m_rows x K, hBt_rows: (N / world) x K (this rank's rows of B^T), hD_rows: m_rows x N, host arrays
        (numpy or torch CPU tensors, pinned for speed). Every rank calls it once per step. Returns when this rank's
        rows of D are in host memory."""
        def addr(x):
            if x is None:
                return None
            return x.data_ptr() if hasattr(x, "data_ptr") else x.ctypes.data
        self.epoch += 1
        st = self.pkg.lib().b200_session_gemm_host_sharded(
            self.session.h, dtype, addr(hA_rows), addr(hBt_rows), addr(hC_rows), addr(hD_rows), alpha, beta, self.m_rows, self.N,
            self.K, self.world, self.rank, self.bt_ptrs, self.flag_ptrs, self.epoch,
            self.C.byref(params) if params is not None else None)
        if st != self.pkg.OK:
            raise self.pkg.B200Error(st, "b200_session_gemm_host_sharded")

    def close(self):
        import torch
        torch.cuda.synchronize()
        self.dist.barrier(group=self.group)
        lib = self.pkg.lib()
        for p in self.imported:
            lib.b200_peer_release(p)
        self.imported = []
        self.dist.barrier(group=self.group)
        if self.flags:
            lib.b200_peer_free(self.flags)
            self.flags = None
        self.session.close()


class PeerLeft(RuntimeError):
    """Raised by Membership.check() when another rank has announced that it left, or has stopped beating."""

    def __init__(self, rank: int, reason: str):
        self.rank, self.reason = rank, reason
        super().__init__(f"rank {rank} left the job: {reason}")


class Membership:
    """Host-side failure detection for the multi-GPU paths, between steps.

    The exchange kernels wait for peers on the device (bounded, with a status record), and a collective
    waits inside NCCL; neither should be entered when a peer is already known to be gone. Every rank
    therefore keeps two notes in the job's key-value store (the TCP store torch.distributed rendezvoused
    on): a heartbeat it refreshes once per step, and a leave note it writes when it goes between steps -
    with none of its kernels or collectives in flight. check(), called before the next launch, raises
    PeerLeft when a peer has left a note or its heartbeat is older than `stale_after` seconds, so the
    survivors stop before they would wait. A peer that dies without a note and inside `stale_after` is
    caught one level down: by the process group's timeout on the next collective, or by the bounded
    wait of the exchange kernel (B200_DEVICE_TIMEOUT). The reference is single-GPU and has nothing of
    the kind (matmul_shmem_tc_async_opt_port_2.cu:1503-1510).
    """

    def __init__(self, store, rank: int, world: int, prefix: str = "b200/members", stale_after: float = 30.0, clock=None):
        import time
        self.store, self.rank, self.world, self.prefix, self.stale_after = store, rank, world, prefix, stale_after
        self.clock = clock or time.time
        self.beat(0)

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def beat(self, step: int) -> None:
        """Refresh this rank's heartbeat (once per step is enough)."""
        self.store.set(self._key("beat", self.rank), f"{step}:{self.clock():.3f}")

    def leave(self, reason: str = "done") -> None:
        """Announce that this rank is going. Call it between steps, after synchronising the device."""
        self.store.set(self._key("left", self.rank), reason)

    def check(self) -> None:
        """Raises PeerLeft if a peer has announced its leave or has not beaten for stale_after seconds."""
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            if self.store.check([self._key("left", r)]):
                raise PeerLeft(r, self.store.get(self._key("left", r)).decode())
            if self.store.check([self._key("beat", r)]):
                _, stamp = self.store.get(self._key("beat", r)).decode().split(":")
                if now - float(stamp) > self.stale_after:
                    raise PeerLeft(r, f"no heartbeat for {now - float(stamp):.1f} s")
