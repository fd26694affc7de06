"""GPU: the split-K entry point that allocates nothing (b200_gemm_splitk_noalloc).

Callers that may not allocate device memory (a serving step that must avoid cudaMalloc's device
synchronisation, a callback under another library's allocator lock, a plugin host with fixed
buffers) get the per-slice partial products stored in a 32 MiB array built into the library.
The result must equal what the regular entry point produces with a caller-provided workspace:
same kernels, same slices, same summation order, so the comparison is exact. Calls in a row
check that the shared array, which keeps the previous call's contents, needs no clearing.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test. It must pass alone in a fresh process and after the other tests.
"""
import numpy as np
import pytest

from helpers import Guarded, inputs, to_device, tolerance_ok

pytestmark = pytest.mark.gpu


def test_no_alloc_split_k_matches_workspace_entry_point_on_calls_in_a_row(pkg, cuda, oracle):
    torch = cuda
    cases = [(pkg.F16, 512, 768, 2048, 4, 1.0, 0.0, 3), (pkg.BF16, 1024, 1024, 1024, 8, 0.5, 2.0, 4)]
    warmed_up = False
    for dtype, m, n, k, split, alpha, beta, seed in cases:
        A, Bt, Cm = inputs(pkg, dtype, m, n, k, 300 + seed)
        dA, dB, dC = to_device(torch, A, dtype), to_device(torch, Bt, dtype), torch.from_numpy(Cm).cuda()
        p = pkg.default_params(m, n, k, dtype, tile_m=128, tile_n=128, split_k=split)
        assert pkg.validate(m, n, k, dtype, p) == pkg.OK
        want = pkg.gemm(dA, dB, dC, None, alpha, beta, p)              # regular entry point, torch-allocated workspace
        assert pkg.device_status()[0] == pkg.OK
        stream = torch.cuda.current_stream().cuda_stream
        gD = Guarded(torch, (m, n), torch.float32)
        got = gD.t
        for call in range(3):                                           # calls in a row share the built-in scratch
            got.fill_(float("nan"))
            torch.cuda.synchronize()
            # Free device memory as the driver reports it (cudaMemGetInfo): unlike torch's own counters it
            # would show a cudaMalloc made inside the library. The very first call on a device may change
            # it (loading this part of the library places the 32 MiB array), later calls must not.
            free_before = torch.cuda.mem_get_info()[0]
            st = pkg.gemm_splitk_noalloc_raw(dtype, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), got.data_ptr(), alpha, beta,
                                             m, n, k, p, stream)
            assert st == pkg.OK, pkg.status_string(st)
            assert pkg.device_status()[0] == pkg.OK
            if warmed_up:
                assert torch.cuda.mem_get_info()[0] == free_before, "free device memory changed across a no-alloc call"
            warmed_up = True
            assert torch.equal(got, want), f"call {call}: built-in scratch and caller workspace disagree"
            gD.check("D of b200_gemm_splitk_noalloc")
        ok, msg = tolerance_ok(want.cpu().numpy(), oracle.gemm(A, Bt, Cm, alpha, beta, dtype), k, abs(alpha) + abs(beta) + 1.0)
        assert ok, msg


def test_no_alloc_rejects_what_does_not_fit(pkg, cuda):
    torch = cuda
    t = torch.zeros(16, dtype=torch.float16, device="cuda")
    d = torch.zeros(16, dtype=torch.float32, device="cuda")
    p = pkg.default_params(4096, 4096, 4096, pkg.F16, tile_m=128, tile_n=128, split_k=2)
    # 2 * 4096 * 4096 values = 128 MiB > 32 MiB built in: refused before anything is launched
    assert pkg.gemm_splitk_noalloc_raw(pkg.F16, t.data_ptr(), t.data_ptr(), None, d.data_ptr(), 1.0, 0.0, 4096, 4096, 4096, p) \
        == pkg.WORKSPACE_TOO_SMALL
    p1 = pkg.default_params(512, 512, 512, pkg.F16, tile_m=128, tile_n=128, split_k=1)
    assert pkg.gemm_splitk_noalloc_raw(pkg.F16, t.data_ptr(), t.data_ptr(), None, d.data_ptr(), 1.0, 0.0, 512, 512, 512, p1) \
        == pkg.INVALID_CONFIG
