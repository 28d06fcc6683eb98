"""nzb_gemm_static: the GEMM entry point that allocates nothing.

Some hosts of this library cannot call cudaMalloc -- a plug-in inside a process whose
framework already owns all device memory, or a steady-state loop where allocation calls
are banned -- so they cannot provide the scratch nzb_gemm wants. nzb_gemm_static keeps
that scratch in a fixed 32 MiB array inside the library. This test drives it through the
C ABI and requires its output to match nzb_gemm's (same kernels, so bit-identical; the
assertion uses the suite's usual e_max <= 2e-5) on two consecutive calls with different
shapes, the second smaller than the first so stale scratch contents would show, checks that the
driver's free-memory figure does not move across the calls (nothing was allocated), reads the path's
own status word, and checks that an oversized problem is refused with a clear message.

Collected last on purpose (file name): a failure here cannot hide other tests from a run
that stops at the first failure. It passes alone in a fresh process and after the rest.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _desc(C, M, N, K):
    d = C.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.lda, d.ldb, d.ldc = K, N, N
    d.batch[0] = d.batch[1] = 1
    return d


def test_static_scratch_gemm_matches_workspace_gemm_twice():
    import neuzephyr_b200 as nz
    from neuzephyr_b200 import _capi as C
    L = C.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cuda")
    g.manual_seed(2024)
    free_seen = []
    for (M, N, K) in [(700, 520, 900), (130, 77, 45), (700, 520, 900)]:
        A = torch.rand((M, K), device="cuda", generator=g) * 2 - 1
        B = torch.rand((K, N), device="cuda", generator=g) * 2 - 1
        bias = torch.rand((N,), device="cuda", generator=g)
        want = nz.gemm(A, B, bias=bias, bias_mode=C.BIAS_ROW, relu=True)
        got = torch.full((M, N), float("nan"), device="cuda")
        d = _desc(C, M, N, K)
        d.bias_mode, d.relu = C.BIAS_ROW, 1
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = L.nzb_gemm_static(ctypes.byref(d), ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(B.data_ptr()),
                               ctypes.c_void_p(got.data_ptr()), ctypes.c_void_p(bias.data_ptr()), stream)
        assert rc == C.OK, L.nzb_last_error_string()
        torch.cuda.synchronize()
        free_seen.append((free_before, torch.cuda.mem_get_info()[0]))
        w, x = want.double().cpu().numpy(), got.double().cpu().numpy()
        assert np.isfinite(x).all()
        assert np.max(np.abs(x - w)) / np.max(np.abs(w)) <= 2e-5
    assert nz.device_status() == 0
    # the first call on a device may make the driver load this library's code and look up the array;
    # from the second call on the free-memory figure must not move at all
    for before, after in free_seen[1:]:
        assert after == before, free_seen
    # the path's own status word (a bounded device-side wait that gave up would be recorded there)
    st = ctypes.c_int(-1)
    assert L.nzb_gemm_static_status(ctypes.byref(st), stream) == C.OK and st.value == 0
    assert L.nzb_gemm_static_status_reset(stream) == C.OK
    assert torch.cuda.mem_get_info()[0] == free_seen[-1][1]


def test_static_scratch_rejects_oversized_problem():
    from neuzephyr_b200 import _capi as C
    L = C.lib()
    d = _desc(C, 4096, 4096, 4096)  # staged operands: 64 MiB > 32 MiB
    need = ctypes.c_size_t(0)
    assert L.nzb_gemm_workspace_bytes(ctypes.byref(d), ctypes.byref(need)) == C.OK
    assert need.value > C.STATIC_SCRATCH_BYTES
    a = torch.zeros(16, device="cuda")
    p = ctypes.c_void_p(a.data_ptr())  # never dereferenced: the size check comes first
    assert L.nzb_gemm_static(ctypes.byref(d), p, p, p, None, None) == C.ERR_WORKSPACE
    msg = L.nzb_last_error_string().decode()
    assert "built-in scratch" in msg and str(C.STATIC_SCRATCH_BYTES) in msg
